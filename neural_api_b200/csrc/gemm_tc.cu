// Dequant-fused GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory) for batches of 9..64 activation rows, where the work is a real dense
// contraction:  Y[b][a] = sum_i W[a][i] * X[b][i],  W = d * code (Q8_0 / Q4_0).
//
// One CTA owns 128 weight rows (the UMMA M dimension) and walks K in chunks of 64:
//   * four warps dequantize the chunk (128 rows x 64 codes) to fp32 exactly, split every
//     value into two bf16 limbs (hi = bf16(v), lo = bf16(v - hi)) and write both as K-major
//     UMMA operand tiles in shared memory (8x16-byte core matrices, no swizzle); the
//     activations are split the same way;
//   * one thread issues, per 16-wide K step, three MMAs  A_hi*B_hi + A_hi*B_lo + A_lo*B_hi
//     (the lo*lo term is below 2^-16 relative) into one fp32 accumulator tile of N = batch
//     columns in tensor memory, then commits to an mbarrier;
//   * two operand stages, so the dequantization of chunk i+1 overlaps the MMAs of chunk i;
//   * the epilogue reads the accumulators with tcgen05.ld (lane = weight row, column =
//     batch row) and applies bias / residual / activation before storing y[b][a].
//   * the tensor core adds into its fp32 accumulator with truncation, which biases long sums towards
//     zero (measured 2.3e-4 relative at K = 27648 in one accumulator); so every TC_FLUSH chunks
//     (K = 512) the accumulator tile is read out and added, rounded to nearest, into fp32 registers,
//     and the next MMA starts a fresh accumulator;
// Relative error against fp32 arithmetic is ~1e-5 per product, far inside the 1e-3 logit
// budget; the exact CUDA-core GEMV stays the path for batches up to 8.
//
// Every mbarrier wait is bounded; tensor memory is freed on every exit path.
#include "gemv_common.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int TC_M = 128;            // weight rows per CTA = UMMA M
constexpr int TC_KC = 64;            // K per chunk (4 UMMA K steps of 16)
constexpr int TC_THREADS = 128;
constexpr int TC_FLUSH = 8;           // chunks accumulated in tensor memory before the read-out into registers
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8 rows x 16 bytes core matrices.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (between the two K core matrices)
//   bits [32,46) stride byte offset >> 4 (between 8-row groups)   bits [46,48) version = 1   bits [61,64) layout = 0
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// Instruction descriptor, kind::f16: D = F32 (bits [4,6) = 1), A = B = BF16 (bits [7,10) = [10,13) = 1),
// both K-major (bits 15, 16 = 0), N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct TcParams {
  const void* codes;
  const __half* scales;
  const float* bias;
  const float* x;
  int64_t ldx;
  float* y;
  int64_t ldy;
  const float* resid;
  int64_t n, k, sstride;
  int batch, nb;       // nb = batch rounded up to 16 (UMMA N)
  int act, epi;
  int* err_flag;
};

// value -> (hi, lo) bf16 limbs, two values packed per 32-bit word
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 ah = __float2bfloat16_rn(a), bh = __float2bfloat16_rn(b);
  const __nv_bfloat16 al = __float2bfloat16_rn(a - __bfloat162float(ah)), bl = __float2bfloat16_rn(b - __bfloat162float(bh));
  hi = (uint32_t)__bfloat16_as_ushort(ah) | ((uint32_t)__bfloat16_as_ushort(bh) << 16);
  lo = (uint32_t)__bfloat16_as_ushort(al) | ((uint32_t)__bfloat16_as_ushort(bl) << 16);
}

template <int TYPE>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const TcParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t mma_bar[2];
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NBP = p.nb;                                   // padded batch = UMMA N
  constexpr int A_BYTES = TC_M * TC_KC * 2;               // one limb of the weight tile: 16 KB
  const int b_bytes = NBP * TC_KC * 2;                    // one limb of the activation tile
  const int stage_bytes = 2 * A_BYTES + 2 * b_bytes;      // A_hi, A_lo, B_hi, B_lo
  constexpr uint32_t LBO = 128, SBO = (TC_KC / 8) * 128;  // core-matrix strides along K / along rows

  // tensor memory: one warp allocates the accumulator columns (a power of two >= 32)
  const uint32_t tmem_cols = NBP <= 32 ? 32u : 64u;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_base_s)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(&mma_bar[0])) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(&mma_bar[1])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_s;

  const int64_t row0 = (int64_t)blockIdx.x * TC_M;
  int64_t my_row = row0 + tid;                            // thread t dequantizes row t of the tile
  if (my_row >= p.n) my_row = p.n - 1;
  const int64_t K = p.k;
  const int64_t row_bytes = (TYPE == CAI_TYPE_Q8_0) ? K : (K >> 1);
  const unsigned char* wrow = (const unsigned char*)p.codes + my_row * row_bytes;
  const unsigned short* srow = (const unsigned short*)p.scales + my_row * p.sstride;
  const uint32_t idesc = umma_idesc(TC_M, NBP);
  const int n_chunks = (int)((K + TC_KC - 1) / TC_KC);    // K is a multiple of 32: the last chunk may be half

  float acc[64];                                          // this thread's weight row x up to 64 batch columns
#pragma unroll
  for (int j = 0; j < 64; ++j) acc[j] = 0.f;

  bool alive = true;
  for (int c = 0; c < n_chunks; ++c) {
    const int stage = c & 1;
    unsigned char* st = smem + (size_t)stage * stage_bytes;
    // the MMAs that read this stage two chunks ago must be done before it is overwritten
    if (c >= 2 && alive && !tc_mbar_wait(tc_smem_u32(&mma_bar[stage]), ((c >> 1) - 1) & 1)) {
      alive = false;
      if (lane == 0) *p.err_flag = 1;
    }
    const int64_t k0 = (int64_t)c * TC_KC;
    const int klen = (int)((K - k0 < TC_KC) ? (K - k0) : TC_KC);     // 64 or 32

    // ---- weights: row `tid`, 64 codes -> fp32 -> bf16 hi/lo -> 8 x 16-byte core-matrix rows per limb ----
    {
      float v[TC_KC];
      if (TYPE == CAI_TYPE_Q8_0) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {                     // two 32-blocks
          if (q * 32 < klen) {
            const float d = __half2float(__ushort_as_half(srow[(k0 >> 5) + q]));
            const int4 w0 = *(const int4*)(wrow + k0 + q * 32), w1 = *(const int4*)(wrow + k0 + q * 32 + 16);
            const uint32_t ww[8] = {(uint32_t)w0.x, (uint32_t)w0.y, (uint32_t)w0.z, (uint32_t)w0.w,
                                    (uint32_t)w1.x, (uint32_t)w1.y, (uint32_t)w1.z, (uint32_t)w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
              for (int j = 0; j < 4; ++j) v[q * 32 + i * 4 + j] = d * (float)((int)((ww[i] >> (8 * j)) & 0xFF) - 128);   // biased codes
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[q * 32 + i] = 0.f;
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (q * 32 < klen) {
            const float d = __half2float(__ushort_as_half(srow[(k0 >> 5) + q]));
            const int4 w0 = *(const int4*)(wrow + ((k0 + q * 32) >> 1));
            const uint32_t ww[4] = {(uint32_t)w0.x, (uint32_t)w0.y, (uint32_t)w0.z, (uint32_t)w0.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t byte = (ww[i] >> (8 * j)) & 0xFF;       // byte e: element e (low), element e+16 (high)
                v[q * 32 + i * 4 + j] = d * (float)((int)(byte & 0x0F) - 8);
                v[q * 32 + 16 + i * 4 + j] = d * (float)((int)(byte >> 4) - 8);
              }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[q * 32 + i] = 0.f;
          }
        }
      }
      const int m8 = tid >> 3, r8 = tid & 7;
#pragma unroll
      for (int k8 = 0; k8 < TC_KC / 8; ++k8) {
        uint4 hi, lo;
        split2(v[k8 * 8 + 0], v[k8 * 8 + 1], hi.x, lo.x);
        split2(v[k8 * 8 + 2], v[k8 * 8 + 3], hi.y, lo.y);
        split2(v[k8 * 8 + 4], v[k8 * 8 + 5], hi.z, lo.z);
        split2(v[k8 * 8 + 6], v[k8 * 8 + 7], hi.w, lo.w);
        const int off = (m8 * (TC_KC / 8) + k8) * 128 + r8 * 16;
        *(uint4*)(st + off) = hi;
        *(uint4*)(st + A_BYTES + off) = lo;
      }
    }
    // ---- activations: (batch row, 8-wide K group) items over the 128 threads ----
    for (int item = tid; item < NBP * (TC_KC / 8); item += TC_THREADS) {
      const int b = item / (TC_KC / 8), k8 = item % (TC_KC / 8);
      float xv[8];
      if (b < p.batch && k8 * 8 < klen) {
        const float4 a = *(const float4*)(p.x + (int64_t)b * p.ldx + k0 + k8 * 8);
        const float4 bq = *(const float4*)(p.x + (int64_t)b * p.ldx + k0 + k8 * 8 + 4);
        xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w; xv[4] = bq.x; xv[5] = bq.y; xv[6] = bq.z; xv[7] = bq.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = 0.f;
      }
      uint4 hi, lo;
      split2(xv[0], xv[1], hi.x, lo.x);
      split2(xv[2], xv[3], hi.y, lo.y);
      split2(xv[4], xv[5], hi.z, lo.z);
      split2(xv[6], xv[7], hi.w, lo.w);
      const int off = ((b >> 3) * (TC_KC / 8) + k8) * 128 + (b & 7) * 16;
      *(uint4*)(st + 2 * A_BYTES + off) = hi;
      *(uint4*)(st + 2 * A_BYTES + b_bytes + off) = lo;
    }
    // make the generic-proxy writes visible to the tensor-core (async) proxy, then hand over
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_hi = tc_smem_u32(st), a_lo = a_hi + A_BYTES, b_hi = a_hi + 2 * A_BYTES, b_lo = b_hi + b_bytes;
#pragma unroll
      for (int ks = 0; ks < TC_KC / 16; ++ks) {
        const uint32_t koff = ks * 2 * 128;               // two core matrices along K per step
        const uint64_t dah = umma_desc(a_hi + koff, LBO, SBO), dal = umma_desc(a_lo + koff, LBO, SBO);
        const uint64_t dbh = umma_desc(b_hi + koff, LBO, SBO), dbl = umma_desc(b_lo + koff, LBO, SBO);
        umma_bf16(tmem_d, dah, dbh, idesc, ((c % TC_FLUSH) != 0 || ks > 0) ? 1u : 0u);   // fresh accumulator after a read-out
        umma_bf16(tmem_d, dah, dbl, idesc, 1u);
        umma_bf16(tmem_d, dal, dbh, idesc, 1u);
      }
      // arrives on the barrier once every MMA issued so far has finished reading shared memory
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem_u32(&mma_bar[stage])) : "memory");
    }
    if ((c % TC_FLUSH) == TC_FLUSH - 1 || c == n_chunks - 1) {
      // read the accumulator tile out: wait for this chunk's commit (it covers every MMA issued so far)
      if (alive && !tc_mbar_wait(tc_smem_u32(&mma_bar[stage]), (c >> 1) & 1)) {
        alive = false;
        if (lane == 0) *p.err_flag = 1;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 16) {
        if (c0 < NBP) {                                   // warp w reads accumulator lanes 32w..32w+31, 16 columns at a time
          uint32_t r[16];
          const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(taddr)
              : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c0 + j] += __uint_as_float(r[j]);
        }
      }
      // the next MMA (fresh accumulator) is issued only after the __syncthreads of the next chunk,
      // which every warp reaches after its loads above have completed
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  }
  // ---- epilogue: thread = weight row, acc[b] = batch column b ----
  const int64_t row = row0 + tid;
  if (row < p.n) {
#pragma unroll
    for (int b = 0; b < 64; ++b) {
      if (b < p.batch) {
        float v = acc[b];
        if (p.bias) v += p.bias[row];
        v = apply_act(v, p.act);
        if (p.epi == EPI_RESID) v += p.resid[(int64_t)b * p.ldy + row];
        p.y[(int64_t)b * p.ldy + row] = v;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
}

}  // namespace

// Launches the tensor-core GEMM, or returns CAI_ERR_UNSUPPORTED (no message) when the call is outside
// what it covers: batches of 9..64 rows, plain or residual epilogue, Q8_0 / Q4_0 weights, no expert indexing.
int gemm_tc_launch(cai_ctx* ctx, const GemvParams& g, int type) {
  if (!ctx->err_flag || g.expert_ids || g.batch < 9 || g.batch > 64) return CAI_ERR_UNSUPPORTED;
  if (g.epi != EPI_STORE && g.epi != EPI_RESID) return CAI_ERR_UNSUPPORTED;
  if (g.norm_gain || g.row_scale) return CAI_ERR_UNSUPPORTED;
  if (((uintptr_t)g.x % 16) || (g.ldx % 4)) return CAI_ERR_UNSUPPORTED;
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.codes = g.codes; p.scales = g.scales; p.bias = g.bias; p.x = g.x; p.ldx = g.ldx; p.y = g.y; p.ldy = g.ldy; p.resid = g.resid;
  p.n = g.n; p.k = g.k; p.sstride = g.sstride; p.batch = g.batch; p.nb = (g.batch + 15) / 16 * 16; p.act = g.act; p.epi = g.epi;
  p.err_flag = ctx->err_flag;
  const size_t smem = 2 * (size_t)(2 * TC_M * TC_KC * 2 + 2 * p.nb * TC_KC * 2);
  const int grid = (int)((g.n + TC_M - 1) / TC_M);
  cudaError_t e;
  if (type == CAI_TYPE_Q8_0) {
    e = cudaFuncSetAttribute(gemm_tc_kernel<CAI_TYPE_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) gemm_tc_kernel<CAI_TYPE_Q8_0><<<grid, TC_THREADS, smem, ctx->stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(gemm_tc_kernel<CAI_TYPE_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) gemm_tc_kernel<CAI_TYPE_Q4_0><<<grid, TC_THREADS, smem, ctx->stream>>>(p);
  }
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "gemm_tc smem attribute -> %s", cudaGetErrorString(e));
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
