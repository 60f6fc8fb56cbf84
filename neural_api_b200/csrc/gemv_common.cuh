// Pieces shared by the quantized GEMV kernels: launch parameters, the exact
// code -> float conversion with packed fp32x2 arithmetic, and the epilogue.
#pragma once
#include "cai_common.cuh"

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
  int64_t sstride;  // halves between scale rows
  int batch;
  int act;
  int epi;
  int ksplit;       // warps cooperating on one row group
  int64_t cta_blocks;   // row blocks of one CTA's worth of rows; CTAs stride over them
  int x_in_smem;    // activations staged in shared memory by the CTA
  int ring_depth;   // stages of the per-warp cp.async ring (ring variant of the kernel), 0 = register prefetch
  int ring_off;     // byte offset of the rings in dynamic shared memory (16-byte aligned)
  // indexed (expert bank) mode
  const void* const* bank_codes;
  const __half* const* bank_scales;
  const int32_t* expert_ids;
  int bank_count;   // expert ids are clamped into [0, bank_count): the ids come from device memory the caller owns
  int x_row_div;
  const float* row_scale;
  const float* out_scale;   // CAI_TYPE_I8ROW: one fp32 scale per weight row, applied to the finished sum (before the bias)
  int* err_flag;    // set by a kernel whose bounded wait ran out
  const float* norm_gain;   // fused per-token RMSNorm of the input (needs x_in_smem), NULL = none
  float norm_eps;
  // EPI_QKV_ROPE
  const float* rope_cs;
  int rope_q_width, rope_kv_width, rope_head_dim, rope_kv_heads, rope_max_ctx;
  int k_blocked;
  float* k_cache;
  float* v_cache;
  const int32_t* cache_len;
};

typedef unsigned long long f32x2_t;   // two packed floats in one 64-bit register

__device__ __forceinline__ f32x2_t pack2(float lo, float hi) {
  f32x2_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float sum2(f32x2_t v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo + hi;
}
// Blackwell packed fp32: two IEEE fp32 operations per instruction (round to nearest even,
// identical results to two scalar operations).
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
  f32x2_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// fp16 bit pattern -> float.
__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)h));      // exact for every half; runs on the conversion pipe
}

// Streaming 16-byte load of weight codes: read-only path, no L1 allocation (each byte is used once).
__device__ __forceinline__ int4 ldg_stream16(const void* ptr) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

// 4 biased Q8_0 codes (q + 128, one per byte) times 4 activations, accumulated into a packed pair.
// (0x4B000000 | byte) is the float 2^23 + q + 128; adding -(2^23 + 128) leaves q exactly.
__device__ __forceinline__ f32x2_t q8_word_fma(uint32_t w, const float4& x, f32x2_t acc) {
  const f32x2_t negc = pack2(-8388736.0f, -8388736.0f);
  const f32x2_t f01 = pack2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651u)));
  const f32x2_t f23 = pack2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652u)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653u)));
  acc = fma2(add2(f01, negc), pack2(x.x, x.y), acc);
  acc = fma2(add2(f23, negc), pack2(x.z, x.w), acc);
  return acc;
}
// 8 nibbles of one 32-bit word of a Q4_0 block: byte e of the block holds element e (low nibble)
// and element e+16 (high nibble); xlo/xhi are the activations of the two element groups.
__device__ __forceinline__ f32x2_t q4_word_fma(uint32_t w, const float4& xlo, const float4& xhi, f32x2_t acc) {
  const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
  const f32x2_t negc = pack2(-8388616.0f, -8388616.0f);   // -(2^23 + 8)
  const f32x2_t l01 = pack2(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7650u)), __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7651u)));
  const f32x2_t l23 = pack2(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7652u)), __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7653u)));
  const f32x2_t h01 = pack2(__uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7650u)), __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7651u)));
  const f32x2_t h23 = pack2(__uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7652u)), __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7653u)));
  acc = fma2(add2(l01, negc), pack2(xlo.x, xlo.y), acc);
  acc = fma2(add2(l23, negc), pack2(xlo.z, xlo.w), acc);
  acc = fma2(add2(h01, negc), pack2(xhi.x, xhi.y), acc);
  acc = fma2(add2(h23, negc), pack2(xhi.z, xhi.w), acc);
  return acc;
}

// Position of activation k (a multiple of 4) in the staged, swizzled row: within each lane segment (16 floats for
// Q8_0, 32 for Q4_0) the 16-byte pieces are XOR-ed with the segment index, so a quarter-warp's reads of piece i
// fall on 8 different bank groups.
template <int TYPE>
__device__ __forceinline__ int64_t x_phys(int64_t k) {
  if (TYPE != CAI_TYPE_Q4_0) return (k & ~(int64_t)12) | ((((k >> 2) & 3) ^ ((k >> 5) & 3)) << 2) | (k & 3);
  return (k & ~(int64_t)28) | ((((k >> 2) & 7) ^ ((k >> 5) & 7)) << 2) | (k & 3);
}

// cp.async pieces of the ring variant (16 bytes, L2 only; a source size of 0 zero-fills the destination)
__device__ __forceinline__ void gv_cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void gv_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most depth-2 of this thread's copy groups are still in flight
__device__ __forceinline__ void gv_cp_async_wait_depth(int depth) {
  if (depth >= 8) asm volatile("cp.async.wait_group 6;" ::: "memory");
  else if (depth == 7) asm volatile("cp.async.wait_group 5;" ::: "memory");
  else if (depth == 6) asm volatile("cp.async.wait_group 4;" ::: "memory");
  else if (depth == 5) asm volatile("cp.async.wait_group 3;" ::: "memory");
  else if (depth == 4) asm volatile("cp.async.wait_group 2;" ::: "memory");
  else if (depth == 3) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else asm volatile("cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ int4 gv_lds16(uint32_t addr) {
  int4 v;
  asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t gv_lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

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
// With resid_fetched, lane r*NB + b already holds the residual element of output (row unit0 + r, batch row b).
template <int NB, int RPW>
__device__ __forceinline__ void gemv_epilogue(const GemvParams& p, const float (&acc)[RPW][NB], int64_t unit0,
                                              int b0, int pair, const float* bias, float resid_pre = 0.f,
                                              bool resid_fetched = false) {
  const int lane = threadIdx.x & 31;
  if (p.epi == EPI_QKV_ROPE) {
    // rows come in (even, odd) pairs = the interleaved RoPE pairs (2k, 2k+1) of a head
    const int hd = p.rope_head_dim, half_hd = hd >> 1;
#pragma unroll
    for (int r = 0; r + 1 < RPW; r += 2) {
      const int64_t row = unit0 + r;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if (lane == ((r * NB + b) & 31) && row + 1 < p.n && (b0 + b) < p.batch) {
          const int bi = b0 + b;
          float v0 = acc[r][b], v1 = acc[r + 1][b];
          if (bias) { v0 += bias[row]; v1 += bias[row + 1]; }
          if (row < p.rope_q_width + p.rope_kv_width) {
            const int64_t rr = (row < p.rope_q_width) ? row : row - p.rope_q_width;
            const float* cs = p.rope_cs + ((size_t)bi * half_hd + (size_t)((rr % hd) >> 1)) * 2;
            const float c = cs[0], s = cs[1];
            const float y0 = c * v0 - s * v1, y1 = s * v0 + c * v1;
            v0 = y0; v1 = y1;
          }
          if (row < p.rope_q_width) {
            p.y[(int64_t)bi * p.ldy + row] = v0;
            p.y[(int64_t)bi * p.ldy + row + 1] = v1;
          } else {
            const bool is_k = row < p.rope_q_width + p.rope_kv_width;
            const int64_t rr = row - p.rope_q_width - (is_k ? 0 : p.rope_kv_width);
            const int64_t g = rr / hd, d = rr % hd;
            const int slot = p.cache_len[bi];
            const int64_t head0 = ((int64_t)bi * p.rope_kv_heads + g) * p.rope_max_ctx * hd;
            float* dst = (is_k ? p.k_cache : p.v_cache) + head0 +
                         ((is_k && p.k_blocked) ? (int64_t)cai_k_blocked_index(slot, (int)d, hd) : (int64_t)slot * hd + d);
            dst[0] = v0; dst[1] = v1;
          }
        }
      }
    }
    return;
  }
  if (p.epi == EPI_SWIGLU) {
    const int64_t half = p.n >> 1;
#pragma unroll
    for (int r = 0; r + 1 < RPW; r += 2) {
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
        if (p.epi == EPI_RESID) v += resid_fetched ? resid_pre : p.resid[yrow * p.ldy + row];
        p.y[yrow * p.ldy + row] = v;
      }
    }
  }
}
