// Device decoders of the ggml block formats (raw file bytes in, fp32 out), shared by the load-time decoder, the
// resident K-quant matrices (dequantization hook, embedding gather) and the K-quant GEMV.
// Block rules: neural/neuralgguf.pas:448-945, 1487-1503.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace ggufdev {

// ---------------------------------------------------------------------------
// device decoders: one thread per output element; every product and sum is rounded on its own (no fused
// multiply-add), which is how the reference's single-precision expressions evaluate
// ---------------------------------------------------------------------------
__device__ __forceinline__ float f16_at(const uint8_t* p) {
  const unsigned short bits = (unsigned short)(p[0] | (p[1] << 8));
  return __half2float(__ushort_as_half(bits));
}

// 6-bit scale and min j of a Q4_K / Q5_K super-block (DequantizeQ4KScaleMin, neural/neuralgguf.pas:448-465)
__device__ __forceinline__ void scale_min_k4(const uint8_t* s, int j, int* sc, int* mn) {
  if (j < 4) {
    *sc = s[j] & 0x3F;
    *mn = s[j + 4] & 0x3F;
  } else {
    const int d = s[j - 4], m = s[j], md = s[j + 4];
    *sc = (md & 0x0F) | ((d >> 2) & 0x30);
    *mn = (md >> 4) | ((m >> 2) & 0x30);
  }
}

__device__ __forceinline__ int legacy_nibble(const uint8_t* qs, int e) {     // LegacyNibble, :811-817
  return e < 16 ? (qs[e] & 0x0F) : (qs[e - 16] >> 4);
}

__device__ __forceinline__ float decode_element(int type, const uint8_t* __restrict__ blk, int e) {
  switch (type) {
    case 2: {                                                                 // Q4_0, :822-845
      const float d = f16_at(blk);
      return __fmul_rn(d, (float)(legacy_nibble(blk + 2, e) - 8));
    }
    case 3: {                                                                 // Q4_1, :850-874
      const float d = f16_at(blk), m = f16_at(blk + 2);
      return __fadd_rn(__fmul_rn(d, (float)legacy_nibble(blk + 4, e)), m);
    }
    case 6: {                                                                 // Q5_0, :879-908
      const float d = f16_at(blk);
      const unsigned qh = blk[2] | (blk[3] << 8) | (blk[4] << 16) | ((unsigned)blk[5] << 24);
      const int q = legacy_nibble(blk + 6, e) | (int)(((qh >> e) & 1u) << 4);
      return __fmul_rn(d, (float)(q - 16));
    }
    case 7: {                                                                 // Q5_1, :913-945
      const float d = f16_at(blk), m = f16_at(blk + 2);
      const unsigned qh = blk[4] | (blk[5] << 8) | (blk[6] << 16) | ((unsigned)blk[7] << 24);
      const int q = legacy_nibble(blk + 8, e) | (int)(((qh >> e) & 1u) << 4);
      return __fadd_rn(__fmul_rn(d, (float)q), m);
    }
    case 8: {                                                                 // Q8_0, :1487-1503
      const float d = f16_at(blk);
      return __fmul_rn((float)(int8_t)blk[2 + e], d);
    }
    case 10: {                                                                // Q2_K, :606-660
      const int sb = e >> 4;
      const int scb = blk[sb];
      const float d = f16_at(blk + 80), dmin = f16_at(blk + 82);
      const float dl = __fmul_rn(d, (float)(scb & 0x0F)), ml = __fmul_rn(dmin, (float)(scb >> 4));
      const int c = e >> 7, s = (e & 127) >> 5, p = e & 31;
      const int q = (blk[16 + c * 32 + p] >> (2 * s)) & 3;
      return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    }
    case 11: {                                                                // Q3_K, :762-806
      const int j = e >> 4;
      const uint8_t* sp = blk + 96;
      int lsc = sp[j & 7];
      lsc = j < 8 ? (lsc & 0x0F) : ((lsc >> 4) & 0x0F);
      const int hsc = (sp[8 + (j & 3)] >> ((j >> 2) * 2)) & 3;
      const int scale = (int)(int8_t)(uint8_t)(lsc | (hsc << 4)) - 32;
      const float dl = __fmul_rn(f16_at(blk + 108), (float)scale);
      const int h0 = e >> 7, s = (e & 127) >> 5, p = e & 31;
      const int ql = (blk[32 + h0 * 32 + p] >> (2 * s)) & 3;
      const int hb = (blk[p] >> (e >> 5)) & 1;
      return __fmul_rn(dl, (float)(ql - ((hb ^ 1) << 2)));
    }
    case 12: {                                                                // Q4_K, :474-520
      const int j = e >> 5, i = e & 31;
      int sc, mn;
      scale_min_k4(blk + 4, j, &sc, &mn);
      const float dl = __fmul_rn(f16_at(blk), (float)sc), ml = __fmul_rn(f16_at(blk + 2), (float)mn);
      const int pb = blk[16 + (j >> 1) * 32 + i];
      const int q = (j & 1) ? (pb >> 4) : (pb & 0x0F);
      return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    }
    case 13: {                                                                // Q5_K, :536-590
      const int j = e >> 5, i = e & 31;
      int sc, mn;
      scale_min_k4(blk + 4, j, &sc, &mn);
      const float dl = __fmul_rn(f16_at(blk), (float)sc), ml = __fmul_rn(f16_at(blk + 2), (float)mn);
      const int pb = blk[48 + (j >> 1) * 32 + i];
      const int q = ((j & 1) ? (pb >> 4) : (pb & 0x0F)) | (((blk[16 + i] >> j) & 1) << 4);
      return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    }
    case 14: {                                                                // Q6_K, :676-738
      const int g = e >> 4;
      const float dl = __fmul_rn(f16_at(blk + 208), (float)(int8_t)blk[192 + g]);
      const int hi = e >> 7, r = e & 127;
      int ql = blk[hi * 64 + (e & 63)];
      ql = r < 64 ? (ql & 0x0F) : (ql >> 4);
      const int qh = (blk[128 + hi * 32 + (e & 31)] >> ((r >> 5) * 2)) & 3;
      return __fmul_rn(dl, (float)((ql | (qh << 4)) - 32));
    }
    default: return 0.f;
  }
}


// ---------------------------------------------------------------------------
// Eight weights of one 256-element super-block for lane `lane` of a warp, as two runs of four consecutive elements
// that start at ea and eb (multiples of 4): the lane's four code bytes carry one run in their low and one in their high
// nibbles. Every weight is formed exactly as the element decoder above forms it (same products, same roundings).
// ---------------------------------------------------------------------------
template <int TYPE> struct KQ;
template <> struct KQ<12> { static constexpr int BB = 144; };
template <> struct KQ<13> { static constexpr int BB = 176; };
template <> struct KQ<14> { static constexpr int BB = 210; };

template <int TYPE>
__device__ __forceinline__ void kq_lane_elements(int lane, int& ea, int& eb) {
  if (TYPE == 14) { ea = (lane >> 4) * 128 + (lane & 15) * 4; eb = ea + 64; }
  else { ea = (lane >> 3) * 64 + (lane & 7) * 4; eb = ea + 32; }
}

// The bytes of a super-block a lane needs, fetched ahead of their use (the GEMV requests the next super-block's before
// it computes on the current one's): Q4_K / Q5_K blocks are 16-byte aligned, so the 16-byte head (d, dmin, the twelve
// packed scale bytes) is one load; Q6_K blocks (210 bytes) are only 2-byte aligned and are read in 16-bit pieces.
struct KQRaw {
  uint4 head;          // Q4_K / Q5_K: bytes 0..15.  Q6_K: x = the two group scales (bytes), y = d (fp16 bits)
  uint32_t q;          // the lane's four code bytes
  uint32_t h;          // Q5_K: its four bytes of the fifth-bit plane.  Q6_K: its four bytes of the high-bit plane
};

template <int TYPE>
__device__ __forceinline__ void kq_fetch(const uint8_t* __restrict__ blk, int lane, KQRaw& r) {
  if (TYPE == 12 || TYPE == 13) {
    r.head = *(const uint4*)blk;
    r.q = *(const uint32_t*)(blk + (TYPE == 12 ? 16 : 48) + 4 * lane);
    r.h = (TYPE == 13) ? *(const uint32_t*)(blk + 16 + (lane & 7) * 4) : 0u;
  } else {
    const int half = lane >> 4, pos = (lane & 15) * 4;
    const int g = half * 8 + (pos >> 4);
    const unsigned short* ql16 = (const unsigned short*)(blk + half * 64 + pos);
    const unsigned short* qh16 = (const unsigned short*)(blk + 128 + half * 32 + (pos & 31));
    r.q = (uint32_t)ql16[0] | ((uint32_t)ql16[1] << 16);
    r.h = (uint32_t)qh16[0] | ((uint32_t)qh16[1] << 16);
    r.head.x = (uint32_t)blk[192 + g] | ((uint32_t)blk[192 + g + 4] << 8);
    r.head.y = (uint32_t)*(const unsigned short*)(blk + 208);
    r.head.z = r.head.w = 0u;
  }
}

// The lane's two runs of a super-block as what the GEMV multiplies with: four codes per run packed one per byte (wa, wb),
// the run's scale dl = d * sc (rounded once, as the reference forms it) and its offset ml = dmin * mn (0 for Q6_K, whose
// codes are centred by `KQ_BIAS` instead):  weight = dl * (code - KQ_BIAS) - ml.
template <int TYPE> struct KQBias { static constexpr float value = 0.f; };
template <> struct KQBias<14> { static constexpr float value = 32.f; };

template <int TYPE>
__device__ __forceinline__ void kq_runs(const KQRaw& r, int lane, uint32_t& wa, uint32_t& wb, float& dla, float& mla, float& dlb, float& mlb) {
  if (TYPE == 12 || TYPE == 13) {
    const int c = lane >> 3;
    const float d = __half2float(__ushort_as_half((unsigned short)(r.head.x & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(r.head.x >> 16)));
    // sub-blocks 2c and 2c+1 (DequantizeQ4KScaleMin): both come from byte pair (2c & 3, (2c & 3) + 1) of the three
    // packed groups; sub-blocks 0..3 use six bits of the first two groups, 4..7 splice the third group in
    const int sh = (2 * c & 3) * 8;
    const uint32_t dd = r.head.y >> sh, mm = r.head.z >> sh, md = r.head.w >> sh;
    int sc0, mn0, sc1, mn1;
    if (c < 2) {
      sc0 = dd & 0x3F; mn0 = mm & 0x3F;
      sc1 = (dd >> 8) & 0x3F; mn1 = (mm >> 8) & 0x3F;
    } else {
      sc0 = (md & 0x0F) | ((dd >> 2) & 0x30); mn0 = ((md >> 4) & 0x0F) | ((mm >> 2) & 0x30);
      sc1 = ((md >> 8) & 0x0F) | ((dd >> 10) & 0x30); mn1 = ((md >> 12) & 0x0F) | ((mm >> 10) & 0x30);
    }
    dla = __fmul_rn(d, (float)sc0); mla = __fmul_rn(dmin, (float)mn0);
    dlb = __fmul_rn(d, (float)sc1); mlb = __fmul_rn(dmin, (float)mn1);
    wa = r.q & 0x0F0F0F0Fu;
    wb = (r.q >> 4) & 0x0F0F0F0Fu;
    if (TYPE == 13) {                                    // the fifth bit of sub-block j is bit j of the plane's byte
      wa |= ((r.h >> (2 * c)) & 0x01010101u) << 4;
      wb |= ((r.h >> (2 * c + 1)) & 0x01010101u) << 4;
    }
  } else {
    const int pos = (lane & 15) * 4;
    const float d = __half2float(__ushort_as_half((unsigned short)r.head.y));
    dla = __fmul_rn(d, (float)(int8_t)(r.head.x & 0xFF)); dlb = __fmul_rn(d, (float)(int8_t)((r.head.x >> 8) & 0xFF));
    mla = mlb = 0.f;
    const int sh0 = 2 * (pos >> 5), sh1 = sh0 + 4;
    wa = (r.q & 0x0F0F0F0Fu) | (((r.h >> sh0) & 0x03030303u) << 4);
    wb = ((r.q >> 4) & 0x0F0F0F0Fu) | (((r.h >> sh1) & 0x03030303u) << 4);
  }
}

}  // namespace ggufdev
