// Dequant-fused GEMV for GGUF Q8_0 / Q4_0 weights (small batch), plus a generic
// warp-per-row kernel for F32 / F16 weights of any width.
//
//   y[b][a] = epilogue( sum_i W[a][i] * x[b][i] ),  W[a][i] = d(a, i/32) * code(a, i)
//
// The sum is formed per 32-block as d * (sum code*x) in fp32: one multiply by the
// block scale per 16 codes instead of one per code. Codes become floats exactly
// (integer -> float through the 2^23 magic constant), accumulation is fp32, the
// reduction order is fixed (no atomics), so results are reproducible run to run.
//
// Work split: a warp owns RPW output rows and walks K in 512-code (Q8_0) or
// 1024-code (Q4_0) strides, one 16-byte vector load per lane per row; KSPLIT warps
// of a CTA may share the same rows (small-N / large-K shapes) and are combined in
// shared memory in a fixed order.
#include "cai_common.cuh"
#include <stdlib.h>

struct GemvParams {
  const void* codes;
  const __half* scales;
  const float* bias;
  const float* x;
  int64_t ldx;
  float* y;
  int64_t ldy;
  const float* resid;
  int64_t n;        // weight rows
  int64_t k;
  int batch;
  int act;
  int epi;
  int ksplit;       // warps cooperating on one row group
  // indexed (expert bank) mode
  const void* const* bank_codes;
  const __half* const* bank_scales;
  const int32_t* expert_ids;
  int x_row_div;
  const float* row_scale;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == CAI_ACT_RELU) return v > 0.f ? v : 0.f;
  if (act == CAI_ACT_SIGMOID) {
    if (v > 0.f) return 1.0f / (1.0f + expf(-v));
    const float s = expf(v);
    return s / (1.0f + s);
  }
  if (act == CAI_ACT_TANH) return tanhf(v);
  return v;
}
// swish(b) = b * sigmoid(b), two-branch form: exp never overflows.
__device__ __forceinline__ float swish(float b) {
  float sig;
  if (b > 0.f) sig = 1.0f / (1.0f + expf(-b));
  else { const float s = expf(b); sig = s / (1.0f + s); }
  return b * sig;
}

// Writes the outputs of one row group. acc[r][b] are complete sums held by every
// lane; lane `r*NB + b` (mod 32) does the store.
template <int NB, int RPW>
__device__ __forceinline__ void gemv_epilogue(const GemvParams& p, const float (&acc)[RPW][NB], int64_t unit0,
                                              int b0, int pair, const float* bias) {
  const int lane = threadIdx.x & 31;
  if (p.epi == EPI_SWIGLU) {
    const int64_t half = p.n >> 1;
#pragma unroll
    for (int r = 0; r < RPW; r += 2) {
      const int64_t j = unit0 + (r >> 1);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if (lane == ((r * NB + b) & 31) && j < half && (b0 + b) < p.batch) {
          float up = acc[r][b], gate = acc[r + 1][b];
          if (bias) { up += bias[j]; gate += bias[half + j]; }
          const int64_t yrow = p.expert_ids ? pair : (b0 + b);
          p.y[yrow * p.ldy + j] = up * swish(gate);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int64_t row = unit0 + r;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if (lane == ((r * NB + b) & 31) && row < p.n && (b0 + b) < p.batch) {
        float v = acc[r][b];
        if (bias) v += bias[row];
        v = apply_act(v, p.act);
        const int64_t yrow = p.expert_ids ? pair : (b0 + b);
        if (p.row_scale) v *= p.row_scale[yrow];
        if (p.epi == EPI_RESID) v += p.resid[yrow * p.ldy + row];
        p.y[yrow * p.ldy + row] = v;
      }
    }
  }
}

template <int TYPE, int NB, int RPW>
__global__ void __launch_bounds__(256) gemv_quant_kernel(const GemvParams p) {
  extern __shared__ float smem_red[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_cta = blockDim.x >> 5;
  const int groups_per_cta = warps_per_cta / p.ksplit;
  const int group = warp / p.ksplit;
  const int kpart = warp - group * p.ksplit;

  // operand selection
  const char* codes = (const char*)p.codes;
  const __half* scales = p.scales;
  const float* bias = p.bias;
  int b0 = blockIdx.y * NB;
  int pair = 0;
  const float* x = p.x;
  if (p.expert_ids) {
    pair = blockIdx.y;
    const int e = p.expert_ids[pair];
    codes = (const char*)p.bank_codes[e];
    scales = p.bank_scales[e];
    bias = nullptr;
    x = p.x + (int64_t)(pair / p.x_row_div) * p.ldx;
    b0 = 0;
  } else {
    x = p.x + (int64_t)b0 * p.ldx;
  }

  // rows of this warp
  const int64_t gidx = (int64_t)blockIdx.x * groups_per_cta + group;
  int64_t unit0;
  int64_t rows[RPW];
  if (p.epi == EPI_SWIGLU) {
    const int64_t half = p.n >> 1;
    unit0 = gidx * (RPW / 2);
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      int64_t j = unit0 + (r >> 1);
      if (j >= half) j = half - 1;
      rows[r] = (r & 1) ? half + j : j;
    }
  } else {
    unit0 = gidx * RPW;
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      int64_t row = unit0 + r;
      if (row >= p.n) row = p.n - 1;
      rows[r] = row;
    }
  }

  float acc[RPW][NB];
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;

  const int64_t K = p.k;
  const int64_t bpr = K / CAI_QK;

  if (TYPE == CAI_TYPE_Q8_0) {
    // lane chunk: 16 codes = one 16-byte load; two lanes share a block scale
    const int64_t stride = (int64_t)p.ksplit * 512;
#pragma unroll 2
    for (int64_t k0 = ((int64_t)kpart * 32 + lane) * 16; k0 < K; k0 += stride) {
      int4 wv[RPW];
      float d[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        wv[r] = __ldg((const int4*)(codes + rows[r] * K + k0));
        d[r] = __half2float(scales[rows[r] * bpr + (k0 >> 5)]);
      }
      float part[RPW][NB];
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) part[r][b] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 xv[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int bb = (b0 + b < p.batch) ? b : 0;
          xv[b] = __ldg((const float4*)(x + (int64_t)bb * p.ldx + k0 + 4 * i));
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const uint32_t w = ((const uint32_t*)&wv[r])[i] ^ 0x80808080u;
          const float f0 = biased_byte_to_float(w, 0), f1 = biased_byte_to_float(w, 1);
          const float f2 = biased_byte_to_float(w, 2), f3 = biased_byte_to_float(w, 3);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float s = part[r][b];
            s = fmaf(f0, xv[b].x, s); s = fmaf(f1, xv[b].y, s);
            s = fmaf(f2, xv[b].z, s); s = fmaf(f3, xv[b].w, s);
            part[r][b] = s;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b] = fmaf(d[r], part[r][b], acc[r][b]);
    }
  } else {
    // Q4_0: lane chunk = one whole block (16 bytes = 32 nibbles). Byte e carries
    // element e (low nibble) and element e+16 (high nibble).
    const int64_t stride = (int64_t)p.ksplit * 1024;
    const int64_t row_bytes = K >> 1;
#pragma unroll 2
    for (int64_t k0 = ((int64_t)kpart * 32 + lane) * 32; k0 < K; k0 += stride) {
      int4 wv[RPW];
      float d[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        wv[r] = __ldg((const int4*)(codes + rows[r] * row_bytes + (k0 >> 1)));
        d[r] = __half2float(scales[rows[r] * bpr + (k0 >> 5)]);
      }
      float part[RPW][NB];
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) part[r][b] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 xlo[NB], xhi[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int bb = (b0 + b < p.batch) ? b : 0;
          xlo[b] = __ldg((const float4*)(x + (int64_t)bb * p.ldx + k0 + 4 * i));
          xhi[b] = __ldg((const float4*)(x + (int64_t)bb * p.ldx + k0 + 16 + 4 * i));
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const uint32_t w = ((const uint32_t*)&wv[r])[i];
          const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
          const float l0 = ubyte_to_float(lo, 0, 8388616.0f), l1 = ubyte_to_float(lo, 1, 8388616.0f);
          const float l2 = ubyte_to_float(lo, 2, 8388616.0f), l3 = ubyte_to_float(lo, 3, 8388616.0f);
          const float h0 = ubyte_to_float(hi, 0, 8388616.0f), h1 = ubyte_to_float(hi, 1, 8388616.0f);
          const float h2 = ubyte_to_float(hi, 2, 8388616.0f), h3 = ubyte_to_float(hi, 3, 8388616.0f);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float s = part[r][b];
            s = fmaf(l0, xlo[b].x, s); s = fmaf(l1, xlo[b].y, s);
            s = fmaf(l2, xlo[b].z, s); s = fmaf(l3, xlo[b].w, s);
            s = fmaf(h0, xhi[b].x, s); s = fmaf(h1, xhi[b].y, s);
            s = fmaf(h2, xhi[b].z, s); s = fmaf(h3, xhi[b].w, s);
            part[r][b] = s;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b] = fmaf(d[r], part[r][b], acc[r][b]);
    }
  }

  // lanes -> one value per (row, batch)
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[r][b] = warp_sum(acc[r][b]);

  if (p.ksplit > 1) {
    // fixed-order combine of the KSPLIT warps of a group through shared memory
    float* slot = smem_red + (size_t)warp * (RPW * NB);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) slot[r * NB + b] = acc[r][b];
    }
    __syncthreads();
    if (kpart != 0) return;
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float s = 0.f;
        for (int q = 0; q < p.ksplit; ++q) s += smem_red[(size_t)(group * p.ksplit + q) * (RPW * NB) + r * NB + b];
        acc[r][b] = s;
      }
  }
  if (gidx * ((p.epi == EPI_SWIGLU) ? (RPW / 2) : RPW) >= ((p.epi == EPI_SWIGLU) ? (p.n >> 1) : p.n)) return;
  gemv_epilogue<NB, RPW>(p, acc, unit0, b0, pair, bias);
}

// Generic path: F32 / F16 weights, any K (scalar loads), warp per row (pair of rows for SwiGLU).
template <int NB>
__global__ void __launch_bounds__(256) gemv_generic_kernel(const GemvParams p, int type) {
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
    const int e = p.expert_ids[pair];
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
  for (int64_t i = lane; i < p.k; i += 32) {
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

static int env_int(const char* name, int dflt) {
  const char* s = getenv(name);
  return (s && *s) ? atoi(s) : dflt;
}

template <int TYPE, int NB>
static void launch_quant(cai_ctx* ctx, const GemvParams& p, int rpw, dim3 grid, int threads, size_t smem) {
  if (rpw == 4) gemv_quant_kernel<TYPE, NB, 4><<<grid, threads, smem, ctx->stream>>>(p);
  else if (rpw == 2) gemv_quant_kernel<TYPE, NB, 2><<<grid, threads, smem, ctx->stream>>>(p);
  else gemv_quant_kernel<TYPE, NB, 1><<<grid, threads, smem, ctx->stream>>>(p);
}
template <int TYPE>
static void launch_quant_nb(cai_ctx* ctx, const GemvParams& p, int nb, int rpw, dim3 grid, int threads, size_t smem) {
  if (nb == 1) launch_quant<TYPE, 1>(ctx, p, rpw, grid, threads, smem);
  else if (nb == 2) launch_quant<TYPE, 2>(ctx, p, rpw, grid, threads, smem);
  else if (nb == 4) launch_quant<TYPE, 4>(ctx, p, rpw, grid, threads, smem);
  else launch_quant<TYPE, 8>(ctx, p, rpw, grid, threads, smem);
}

int linear_launch(cai_ctx* ctx, const LinearArgs& a) {
  const QWeight* w = a.w;
  ctx->cur_family = FAM_LINEAR;
  if (!w || !a.x || !a.y) return cai_fail(ctx, CAI_ERR_INVALID, "linear: null operand");
  if (a.batch < 1) return cai_fail(ctx, CAI_ERR_INVALID, "linear: batch %d", a.batch);
  if (a.epilogue == EPI_SWIGLU && (w->n % 2)) return cai_fail(ctx, CAI_ERR_INVALID, "SwiGLU epilogue needs an even row count");
  if (a.epilogue == EPI_RESID && !a.resid) return cai_fail(ctx, CAI_ERR_INVALID, "residual epilogue without residual");
  const bool indexed = a.expert_ids_dev != nullptr;
  GemvParams p;
  p.codes = w->codes; p.scales = w->scales; p.bias = w->bias;
  p.x = a.x; p.ldx = a.ldx; p.y = a.y; p.ldy = a.ldy; p.resid = a.resid;
  p.n = w->n; p.k = w->k; p.batch = a.batch; p.act = a.act; p.epi = a.epilogue;
  p.bank_codes = a.bank_codes_dev; p.bank_scales = a.bank_scales_dev; p.expert_ids = a.expert_ids_dev;
  p.x_row_div = a.x_row_div < 1 ? 1 : a.x_row_div; p.row_scale = a.row_scale_dev;
  p.ksplit = 1;
  const int64_t units = (a.epilogue == EPI_SWIGLU) ? w->n / 2 : w->n;
  const bool quant = (w->type == CAI_TYPE_Q8_0 || w->type == CAI_TYPE_Q4_0);
  if (!quant) {
    const int threads = 128;
    const int wpc = threads / 32;
    const int64_t groups = (a.epilogue == EPI_SWIGLU) ? units : (units + 1) / 2;
    const int nb = indexed ? 1 : (a.batch >= 4 ? 4 : 1);
    dim3 grid((unsigned)((groups + wpc - 1) / wpc), indexed ? a.batch : (unsigned)((a.batch + nb - 1) / nb));
    if (nb == 4) gemv_generic_kernel<4><<<grid, threads, 0, ctx->stream>>>(p, w->type);
    else gemv_generic_kernel<1><<<grid, threads, 0, ctx->stream>>>(p, w->type);
    CAI_LAUNCHED(ctx);
    return CAI_OK;
  }
  if ((a.ldx % 4) || ((uintptr_t)a.x % 16)) return cai_fail(ctx, CAI_ERR_INVALID, "linear: activations must be 16-byte aligned with ldx %% 4 == 0");
  // batch tile
  int nb = 1;
  if (!indexed) nb = a.batch >= 5 ? 8 : (a.batch >= 3 ? 4 : (a.batch == 2 ? 2 : 1));
  // rows per warp / warps per row group: enough 16-byte loads in flight per SM without
  // leaving SMs idle on small matrices
  const int64_t lane_chunk = (w->type == CAI_TYPE_Q8_0) ? 16 : 32;
  const int64_t k_iters_1 = (w->k + lane_chunk * 32 - 1) / (lane_chunk * 32);   // iterations of one warp alone
  int rpw, ksplit;
  const int64_t target_groups = (int64_t)ctx->sm_count * 16;   // warps' worth of row groups for a full machine
  if (units >= target_groups * 4) rpw = 4;
  else if (units >= target_groups * 2) rpw = 2;
  else rpw = (a.epilogue == EPI_SWIGLU) ? 2 : 1;
  if (nb == 8 && rpw == 4) rpw = 2;
  {
    const int64_t groups = (units + ((a.epilogue == EPI_SWIGLU) ? rpw / 2 : rpw) - 1) / ((a.epilogue == EPI_SWIGLU) ? rpw / 2 : rpw);
    ksplit = 1;
    while (ksplit < 8 && groups * ksplit < target_groups && k_iters_1 >= 2 * ksplit) ksplit *= 2;
  }
  rpw = env_int("CAI_GEMV_RPW", rpw);
  ksplit = env_int("CAI_GEMV_KSPLIT", ksplit);
  if (rpw != 1 && rpw != 2 && rpw != 4) rpw = 2;
  if (a.epilogue == EPI_SWIGLU && rpw == 1) rpw = 2;
  if (ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) ksplit = 1;
  p.ksplit = ksplit;
  const int threads = 256;
  const int wpc = threads / 32;
  const int groups_per_cta = wpc / ksplit;
  const int units_per_group = (a.epilogue == EPI_SWIGLU) ? rpw / 2 : rpw;
  const int64_t groups = (units + units_per_group - 1) / units_per_group;
  dim3 grid((unsigned)((groups + groups_per_cta - 1) / groups_per_cta), indexed ? a.batch : (unsigned)((a.batch + nb - 1) / nb));
  const size_t smem = (ksplit > 1) ? (size_t)wpc * rpw * nb * sizeof(float) : 0;
  if (w->type == CAI_TYPE_Q8_0) launch_quant_nb<CAI_TYPE_Q8_0>(ctx, p, nb, rpw, grid, threads, smem);
  else launch_quant_nb<CAI_TYPE_Q4_0>(ctx, p, nb, rpw, grid, threads, smem);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
