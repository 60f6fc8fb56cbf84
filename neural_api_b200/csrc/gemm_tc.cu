// Dequant-fused GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory) for batches of 9..64 activation rows, where the work is a real dense
// contraction:  Y[b][a] = sum_i W[a][i] * X[b][i],  W = d * code (Q8_0 / Q4_0). (Batches of 3..8 rows
// come here too when the matrix is large: the CUDA-core kernel's 8-row tile is slower.)
//
// The block scale d varies along K, so it cannot ride inside one long tensor-core
// accumulation without rounding d * code to 16 bits. Instead the MMA runs on the integer
// codes, which fp16 holds exactly, and each 32-wide block gets its own accumulator:
//
//   split kernel   every activation row is scaled by a power of two into fp16's range and split
//                  once per call into two fp16 limbs (x = x0 + x1, each limb the fp16 rounding of
//                  what is left: 22 significant bits), written in the tile order the MMA reads
//                  (K-major rows of 128 bytes, 128-byte swizzle), so every CTA of the GEMM just copies its tiles;
//   GEMM kernel    one CTA owns 128 weight rows (UMMA M) and walks K in chunks of 64 (two blocks):
//     * 8 worker warps stream the raw code bytes into a shared-memory ring with cp.async (a stage is a run of
//       128..512 contiguous bytes of each row), turn each chunk into fp16 integers laid out as the UMMA A tile
//       (one byte-permute and one packed subtract per two codes), and read the accumulators of the previous
//       chunk out of tensor memory (tcgen05.ld: lane = weight row, column = batch row), adding d * partial
//       into fp32 registers with one FMA per value, rounded to nearest;
//     * a ninth warp (one lane) copies the activation tiles in with bulk copies and issues, per 32-block,
//       2 K-steps x 2 limbs MMAs (fp16 codes x fp16 limbs -> fp32, every product exact) into that block's own
//       accumulator (two chunks = four accumulators in flight), committing each chunk to an mbarrier.
//   So the weights enter exactly, the per-block sums are short (the tensor core adds into its accumulator with
//   truncation, which biases long sums towards zero: 2.3e-4 relative was measured for K = 27648 kept in one
//   accumulator), and the only approximation left is the limb split of the activations, 2^-22 relative:
//   measured error against float64 is ~1e-6 of the output RMS, the same as fp32 arithmetic.
//
//   What bounds it: instruction issue, not the tensor pipe (3 % busy) - unpacking a byte costs more than
//   multiplying it - so everything whose value is known when the kernel is compiled is a template parameter, and
//   the per-thread addressing is hoisted out of the chunk loop.
//
// Every mbarrier wait is bounded; tensor memory is freed on every exit path.
#include "gemv_common.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int TC_M = 128;            // weight rows per CTA = UMMA M
constexpr int TC_KC = 64;            // K per chunk: two 32-blocks, four UMMA K steps of 16
constexpr int TC_DEPTH = 3;          // weight tiles / accumulator sets in flight between conversion and read-out
constexpr int TC_RAW_STAGES = 2;     // ring of raw-code stages
constexpr int TC_A_BYTES = TC_M * TC_KC * 2;  // fp16 weight tile: 16 KB
constexpr uint32_t TC_SPIN_LIMIT = 1u << 20;

// Per batch width (rows rounded up to 16, 32 or 64): worker threads, raw bytes per row and ring stage, depth of the
// activation ring. Two CTAs share an SM up to 32 rows (<= 112 KB and 256 tensor-memory columns each); 64 rows take
// the SM alone with twice the worker warps.
template <int NB> struct TcPlan {
  static constexpr int WORKERS = NB <= 32 ? 256 : 512;
  static constexpr int THREADS = WORKERS + 32 * (TC_DEPTH + 1);                 // plus one MMA warp per accumulator set and the activation-tile warp
  static constexpr int SPAN = NB <= 32 ? 128 : 256;
  static constexpr int B_STAGES = NB == 32 ? 3 : 4;
  static constexpr int B_BYTES = 2 * NB * 128;                                  // two limbs of NB rows x 128 bytes
  static constexpr int SMEM = 1024 + TC_DEPTH * TC_A_BYTES + B_STAGES * B_BYTES + TC_RAW_STAGES * TC_M * SPAN;
  static constexpr int ACC_STRIDE = NB < 32 ? 32 : NB;                          // accumulators start on multiples of 32 columns
  static constexpr int TMEM_COLS = NB <= 32 ? 256 : 512;                        // >= TC_DEPTH * 2 * ACC_STRIDE, a power of two
  static constexpr int MIN_CTAS = NB <= 32 ? 2 : 1;
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bounded wait on an mbarrier phase for the worker warps: poll, and between polls step aside for a few dozen
// nanoseconds so that waiting warps do not crowd the issue slots of the working ones. (try_wait's own
// suspend-time hint is no use here: measured on B200, a hinted try_wait on an incomplete phase came back only
// after the full hinted time, 4 us for a hint of 4000.)
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
    __nanosleep(32);
  }
  return false;
}

// The same wait for the single issuing lanes, with a shorter pause: they should notice completion quickly, but a
// lane that polls without pause keeps the shared-memory pipeline busy, and every shared-memory instruction of the
// working warps (loads, stores, arrivals) queues behind its polls.
__device__ __forceinline__ bool tc_mbar_spin(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < TC_SPIN_LIMIT * 4u; ++i) {
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
    __nanosleep(20);
  }
  return false;
}

// 16-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros without reading.
__device__ __forceinline__ void tc_cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void tc_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tc_cp_async_wait(int pending) {
  if (pending >= 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
  else if (pending == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile in the 128-byte swizzled layout: row r of the tile
// (64 fp16 = 128 bytes) starts at r * 128, and its 16-byte piece j sits at position j ^ (r & 7); tiles start on
// 1024-byte boundaries. (The unswizzled core-matrix layout measured ~250 cycles per 128x16x16 MMA here whatever
// N was: the operand fetch ran at a fraction of the shared-memory bandwidth.)
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (1 for swizzled K-major)
//   bits [32,46) stride byte offset >> 4 = 1024 / 16 between 8-row groups   bits [46,48) version = 1
//   bits [61,64) layout = 2 (128-byte swizzle).  A K step of 16 elements advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16: D = F32 (bits [4,6) = 1), A = B = F16 (bits [7,10) = [10,13) = 0),
// both K-major (bits 15, 16 = 0), N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The four MMAs of one 32-block (two K steps of 16 x two activation limbs) into one fresh accumulator, from the low
// and high words of the A and B descriptors of the block's first K step. Only the start-address field (low word, units
// of 16 bytes) differs between them: +2 for the second K step, +limb for the second limb. One asm statement, so the
// lone issuing thread spends a handful of instructions per MMA.
__device__ __forceinline__ void umma_block(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t limb,
                                           uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      ".reg .b64 a0, a1, b0, b1, b2, b3;\n"
      ".reg .b32 t0, t1, t2, t3;\n"
      "setp.ne.b32 p0, %0, %0;\n"
      "setp.eq.b32 p1, %0, %0;\n"
      "mov.b64 a0, {%1, %2};\n"
      "add.u32 t0, %1, 2;\n"
      "mov.b64 a1, {t0, %2};\n"
      "mov.b64 b0, {%3, %4};\n"
      "add.u32 t1, %3, %5;\n"
      "mov.b64 b1, {t1, %4};\n"
      "add.u32 t2, %3, 2;\n"
      "mov.b64 b2, {t2, %4};\n"
      "add.u32 t3, t1, 2;\n"
      "mov.b64 b3, {t3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a0, b0, %6, p0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a0, b1, %6, p1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b2, %6, p1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b3, %6, p1;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(limb), "r"(idesc)
      : "memory");
}

struct TcParams {
  const unsigned char* codes;
  const __half* scales;
  const float* bias;
  const unsigned char* xp;   // activations, split into limbs and tiled by the split kernel
  const float* row_unscale;  // per batch row: the power of two that undoes the split kernel's scaling
  float* y;
  int64_t ldy;
  const float* resid;
  int64_t n, k, sstride;
  int batch;
  int act, epi;
  int* err_flag;
  // K split over blockIdx.y (matrices with few row tiles): CTA (x, y) handles chunks [y * chunks_per_split, ...)
  // and, when ksplit > 1, stores its unscaled-by-nothing partial sums to part[y][b][row] for the reduce kernel.
  int ksplit, chunks_per_split;
  float* part;
  // Grouped (mixture-of-experts) mode, 16-row tiles: blockIdx.z = tile t. The tile's weights are bank[tile_expert[t]]
  // (t is skipped when that is negative), column b of the tile is pair tile_pairs[16 t + b] (negative = unused), whose
  // result goes to output row `pair`; the tile's split activations start at xp + t * xp_tile_bytes and its row
  // factors at row_unscale + 16 t.
  const int32_t* tile_expert;
  const int32_t* tile_pairs;
  const void* const* bank_codes;
  const __half* const* bank_scales;
  size_t xp_tile_bytes;
};

// ---------------------------------------------------------------------------
// Activation split. One CTA per (padded) batch row; optional RMSNorm of the row first
// (inv = 1/sqrt(mean(x^2) + eps), value = gain * (x * inv), the arithmetic of the norm kernel).
// The row is scaled by a power of two so that its largest magnitude lies in [2^13, 2^14) (exact; keeps
// every limb inside fp16's range, and the small limbs out of its subnormals), then split into fp16
// limbs; the GEMM multiplies the row's results by the inverse factor, also exactly.
// Output: for every 64-wide K chunk, `limbs` tiles of nb rows x 64 fp16 in the swizzled K-major
// layout of the MMA: byte offset row * 128 + ((k8 ^ (row & 7)) * 16) for the 8 values of K group k8.
// Rows beyond the batch and columns beyond K are zeros.
// ---------------------------------------------------------------------------
__global__ void tc_split_x_kernel(const float* __restrict__ x, int64_t ldx, int batch, int nb, int64_t k, int n_chunks, int limbs,
                                  const float* __restrict__ norm_gain, float norm_eps, unsigned char* __restrict__ xp,
                                  float* __restrict__ row_unscale, const int32_t* __restrict__ tile_pairs, int x_row_div,
                                  size_t xp_tile_bytes) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();                     // the previous GEMM may still be reading the tile buffer this kernel rewrites
  const int b = blockIdx.x;
  // grouped mode: tile blockIdx.y gathers its rows through tile_pairs (row of pair p = p / x_row_div)
  int src_row = b;
  bool have = b < batch;
  if (tile_pairs) {
    const int t = blockIdx.y;
    if (tile_pairs[(size_t)t * nb] < 0) return;           // pairs fill a tile from slot 0: an empty first slot = an unused tile
    const int pr = tile_pairs[(size_t)t * nb + b];
    have = pr >= 0;
    src_row = have ? pr / x_row_div : 0;
    xp += (size_t)t * xp_tile_bytes;
    row_unscale += (size_t)t * nb;
  }
  const float* xr = x + (int64_t)src_row * ldx;
  float inv = 1.f, scale = 1.f;
  if (have) {
    if (norm_gain) {
      float ss = 0.f;
      for (int64_t c = threadIdx.x; c < k; c += blockDim.x) { const float v = xr[c]; ss = fmaf(v, v, ss); }
      ss = block_sum(ss, red);
      inv = 1.0f / sqrtf(ss / (float)k + norm_eps);
    }
    float mx = 0.f;
    for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
      const float v = norm_gain ? norm_gain[c] * (xr[c] * inv) : xr[c];
      mx = fmaxf(mx, fabsf(v));
    }
    mx = block_max(mx, red);
    int e = 0;
    if (mx > 0.f && mx < 3.0e38f) e = 13 - ilogbf(mx);     // mx * 2^e in [2^13, 2^14)
    if (e > 100) e = 100;
    if (e < -100) e = -100;
    scale = ldexpf(1.f, e);
    if (threadIdx.x == 0) row_unscale[b] = ldexpf(1.f, -e);
  } else if (threadIdx.x == 0) {
    row_unscale[b] = 0.f;
  }
  const size_t limb_bytes = (size_t)nb * 128, chunk_bytes = (size_t)limbs * limb_bytes;
  for (int g = threadIdx.x; g < n_chunks * 8; g += blockDim.x) {
    const int c = g >> 3, k8 = g & 7;
    const int64_t kk = (int64_t)c * TC_KC + k8 * 8;
    float v[8];
    if (have && kk < k) {                                 // K is a multiple of 32: a group of 8 is whole or absent
      const float4 a0 = *(const float4*)(xr + kk), a1 = *(const float4*)(xr + kk + 4);
      v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
      if (norm_gain) {
        const float4 g0 = *(const float4*)(norm_gain + kk), g1 = *(const float4*)(norm_gain + kk + 4);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = gg[i] * (v[i] * inv);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= scale;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    unsigned char* dst = xp + (size_t)c * chunk_bytes + (size_t)(b * 128 + ((k8 ^ (b & 7)) * 16));
    for (int l = 0; l < limbs; ++l) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half h0 = __float2half_rn(v[2 * i]), h1 = __float2half_rn(v[2 * i + 1]);
        v[2 * i] -= __half2float(h0);                     // exact: the limb is the leading bits of the value
        v[2 * i + 1] -= __half2float(h1);
        w[i] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
      }
      *(uint4*)(dst + (size_t)l * limb_bytes) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// two bytes of `w` (selected by `sel`) -> two fp16 integers 1024 + byte, minus `bias2` (packed fp16): exact
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t w, uint32_t sel, uint32_t bias2) {
  uint32_t h;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(w), "r"(0x64646464u), "r"(sel));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h) : "r"(h), "r"(bias2));
  return h;
}

__device__ __forceinline__ uint4 tc_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void tc_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// reads this thread's lane of NCOL consecutive accumulator columns (NCOL = 8, 16 or 32)
template <int NCOL>
__device__ __forceinline__ void tc_tmem_ld(uint32_t taddr, uint32_t* r) {
  if (NCOL == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
  } else if (NCOL == 16) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
  } else {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, "
        "%19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
  }
}

template <int TYPE, int NB>
__global__ void __launch_bounds__(TcPlan<NB>::THREADS, TcPlan<NB>::MIN_CTAS) gemm_tc_kernel(const TcParams p) {
  using Plan = TcPlan<NB>;
  constexpr int W = Plan::WORKERS;                                           // worker threads
  constexpr int D = TC_DEPTH;
  constexpr int SB = Plan::B_STAGES;
  constexpr int SPAN = Plan::SPAN;                                           // raw code bytes per row and stage
  constexpr int PPR = SPAN / 16;                                             // 16-byte pieces per row and stage
  constexpr int PIECES = (TYPE == CAI_TYPE_Q8_0) ? 4 : 2;                    // pieces per row and 64-wide chunk
  constexpr int SUB = PPR / PIECES;                                          // chunks per stage
  constexpr int RAW_BYTES = TC_M * SPAN;
  constexpr int LIMB_BYTES = NB * 128;                                       // one fp16 limb of the activation tile
  constexpr int B_BYTES = Plan::B_BYTES;
  constexpr int ACC_STRIDE = Plan::ACC_STRIDE;
  constexpr int NCOL = NB / (W / 128);                                       // batch columns a worker thread owns

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t mma_bar[D];            // MMAs of chunk c done (tcgen05.commit), c % D
  __shared__ __align__(8) uint64_t a_ready[D];            // weight tile of chunk c converted (one arrival per worker warp), c % D
  __shared__ __align__(8) uint64_t b_full[SB];            // activation tile landed (bytes of a bulk copy)
  __shared__ __align__(8) uint64_t b_empty[SB];           // the MMAs that read the activation tile are done (tcgen05.commit)
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Programmatic dependent launch: this kernel may start while its predecessor drains. Tensor-memory allocation,
  // barrier set-up and the first stages of weight codes do not depend on it; every role waits (pdl_wait) before it
  // touches what the predecessor wrote (activation tiles, row factors, residual, the tile lists of a grouped call).
  pdl_trigger();
  if (p.tile_expert) pdl_wait();
  // operands: the call's matrix, or in grouped mode the expert matrix and activation tile of tile blockIdx.z
  const unsigned char* w_codes = p.codes;
  const __half* w_scales = p.scales;
  const unsigned char* x_tiles = p.xp;
  const float* unscale = p.row_unscale;
  const int32_t* out_rows = nullptr;                       // grouped: output row of each tile column
  if (p.tile_expert) {
    const int t = blockIdx.z;
    const int e = p.tile_expert[t];
    if (e < 0) return;                                     // unused tile: the whole CTA leaves before touching anything
    w_codes = (const unsigned char*)p.bank_codes[e];
    w_scales = p.bank_scales[e];
    x_tiles += (size_t)t * p.xp_tile_bytes;
    unscale += (size_t)t * NB;
    out_rows = p.tile_pairs + (size_t)t * NB;
  }
  // operand tiles start on 1024-byte boundaries (the swizzle works on absolute shared-memory address bits)
  const uint32_t smem0 = (tc_smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_st = smem0;                                               // D tiles of 16 KB
  const uint32_t b_st = a_st + D * TC_A_BYTES;                               // SB tiles, each a multiple of 1 KB
  const uint32_t raw_st = b_st + SB * B_BYTES;                               // TC_RAW_STAGES stages

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_base_s)), "r"((uint32_t)Plan::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < D; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(&mma_bar[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem_u32(&a_ready[i])), "r"(W / 32) : "memory");
    }
    for (int i = 0; i < SB; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(&b_full[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(&b_empty[i])) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_s;

  const int64_t row0 = (int64_t)blockIdx.x * TC_M;
  const int64_t K = p.k;
  const int64_t row_bytes = (TYPE == CAI_TYPE_Q8_0) ? K : (K >> 1);
  // this CTA's K range: chunks [chunk0, chunk0 + n_chunks) of the row (chunk0 is a multiple of 8, so raw stages
  // and the 16-byte groups of scales stay aligned); the row's last chunk may be half (K is a multiple of 32)
  const int chunk0 = (int)blockIdx.y * p.chunks_per_split;
  const int total_chunks = (int)((K + TC_KC - 1) / TC_KC);
  const int n_chunks = (total_chunks - chunk0 < p.chunks_per_split) ? (total_chunks - chunk0) : p.chunks_per_split;
  const int n_blocks = (int)(K >> 5) - 2 * chunk0;        // blocks from chunk0 to the end of the row
  const int n_stages = (n_chunks + SUB - 1) / SUB;
  const int64_t kbyte0 = (int64_t)chunk0 * (TYPE == CAI_TYPE_Q8_0 ? TC_KC : TC_KC / 2);   // first code byte of the range within a row

  if (warp == W / 32 + D) {
    // =====================================================================================
    // Activation-tile warp (one lane): one bulk copy per chunk (the split kernel wrote the tile in the layout the
    // MMA reads) into ring slot j % SB, completion counted in bytes on that slot's mbarrier; a slot is refilled once
    // the MMAs that read it are done.
    // =====================================================================================
    if (lane == 0) {
      pdl_wait();                                           // the tiles are the split kernel's output
      const uint32_t bar_f = tc_smem_u32(&b_full[0]), bar_e = tc_smem_u32(&b_empty[0]);
      int slot = 0;
      uint32_t eparity = 1;                                 // parity of the "emptied" phase awaited: none on the first lap
      const unsigned char* src = x_tiles + (size_t)chunk0 * B_BYTES;
      for (int j = 0; j < n_chunks; ++j) {
        if (j >= SB && !tc_mbar_wait(bar_e + 8u * slot, eparity)) { *p.err_flag = 1; break; }
        const uint32_t bar = bar_f + 8u * (uint32_t)slot;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)B_BYTES) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         b_st + (uint32_t)(slot * B_BYTES)),
                     "l"(src), "r"((uint32_t)B_BYTES), "r"(bar)
                     : "memory");
        src += B_BYTES;
        if (++slot == SB) { slot = 0; eparity ^= 1; }
      }
    }
  } else if (warp >= W / 32) {
    // =====================================================================================
    // MMA warps (one lane each), one per accumulator set: warp s issues the chunks c = s, s + D, ... A lone thread
    // runs slowly on a busy SM (measured ~1600 cycles for the waits, the eight MMAs and the commits of one chunk),
    // so the chunks are dealt out over D issuing threads.
    // =====================================================================================
    if (lane == 0) {
      bool alive = true;
      const int set = warp - W / 32;
      const uint32_t idesc = umma_idesc(TC_M, NB);
      const uint64_t da0 = umma_desc(a_st + (uint32_t)(set * TC_A_BYTES)), db0 = umma_desc(b_st);
      const uint32_t a_lo = (uint32_t)da0, a_hi = (uint32_t)(da0 >> 32), b_lo0 = (uint32_t)db0, b_hi = (uint32_t)(db0 >> 32);
      const uint32_t bar_mma = tc_smem_u32(&mma_bar[set]), bar_a = tc_smem_u32(&a_ready[set]);
      const uint32_t bar_f = tc_smem_u32(&b_full[0]), bar_e = tc_smem_u32(&b_empty[0]);
      const uint32_t d_t = tmem_d + (uint32_t)(set * 2 * ACC_STRIDE);
      uint32_t aparity = 0;
      for (int c = set; c < n_chunks; c += D) {
        const int bslot = c % SB;
        // weight tile converted (which also says the workers have read out the accumulators of chunk c-D), activation tile landed
        if (alive && !tc_mbar_spin(bar_a, aparity)) { alive = false; *p.err_flag = 1; }
        if (alive && !tc_mbar_spin(bar_f + 8u * bslot, (uint32_t)((c / SB) & 1))) { alive = false; *p.err_flag = 1; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t b_lo = b_lo0 + (uint32_t)((bslot * B_BYTES) >> 4);
        // each 32-block into its own fresh accumulator; the second block starts 64 bytes (4 units) into the rows
        umma_block(d_t, a_lo, a_hi, b_lo, b_hi, (uint32_t)(LIMB_BYTES >> 4), idesc);
        if (2 * c + 1 < n_blocks) umma_block(d_t + ACC_STRIDE, a_lo + 4, a_hi, b_lo + 4, b_hi, (uint32_t)(LIMB_BYTES >> 4), idesc);
        // both arrive once every MMA issued so far by this thread has finished (operands read, accumulators written);
        // the activation slot's barrier only while someone will still wait on it
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_mma) : "memory");
        if (c + SB < n_chunks)
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_e + 8u * bslot) : "memory");
        aparity ^= 1;
      }
    }
  } else {
    // =====================================================================================
    // Worker warps. Read-out role: warp w reads accumulator lanes 32*(w&3).., batch columns [cg*NCOL, (cg+1)*NCOL),
    // cg = w >> 2. Everything that does not change from chunk to chunk is computed here, once.
    // =====================================================================================
    const int lane_q = warp & 3, cg = warp >> 2;
    int64_t my_row = row0 + lane_q * 32 + lane;
    const bool row_ok = my_row < p.n;
    if (!row_ok) my_row = p.n - 1;
    const uint4* srow = (const uint4*)(w_scales + my_row * p.sstride) + (chunk0 >> 2);     // 8 scales (4 chunks) per 16 bytes
    uint4 sc_cur = make_uint4(0, 0, 0, 0), sc_next = srow[0];
    // the running sums of a thread's NCOL batch columns, as packed pairs: one fma.rn.f32x2 adds d * accumulator for two
    // columns (each lane an IEEE fused multiply-add, so the result equals the one-column form bit for bit)
    static_assert(NCOL % 2 == 0, "batch columns per thread come in pairs");
    f32x2_t acc2[NCOL / 2];
#pragma unroll
    for (int j = 0; j < NCOL / 2; ++j) acc2[j] = 0ull;
    bool alive = true;
    const uint32_t bar_mma = tc_smem_u32(&mma_bar[0]), bar_a = tc_smem_u32(&a_ready[0]);
    const uint32_t t_lane = tmem_d + ((uint32_t)(lane_q * 32) << 16) + (uint32_t)(cg * NCOL);
    const int rmax = (int)((p.n - 1 - row0 < TC_M - 1) ? (p.n - 1 - row0) : (TC_M - 1));   // last valid row of the tile

    // ---- raw-code producer. Item i = tid + W t of a stage is 16-byte piece (i % PPR) of row (i / PPR): a thread
    //      keeps its piece and walks down the rows in steps of W / PPR, so source and destination advance by constants.
    //      The pieces of a row are XOR-swizzled with the row, so that the conversion, which walks rows, reads without
    //      bank conflicts (the row step is a multiple of 8, so a thread's swizzle is fixed too).
    constexpr int RSTEP = W / PPR;
    static_assert(RSTEP % 8 == 0, "row step must keep the swizzle fixed");
    const int pr_pc = tid & (PPR - 1), pr_r0 = tid / PPR;
    const uint32_t pr_dst0 = (uint32_t)(pr_r0 * SPAN + ((pr_pc ^ (pr_r0 & 7)) << 4));
    const unsigned char* pr_src0 = w_codes + row0 * row_bytes + kbyte0 + pr_pc * 16;
    auto issue_raw = [&](int j) {
      if (j < n_stages) {
        const uint32_t dst = raw_st + (uint32_t)((j & (TC_RAW_STAGES - 1)) * RAW_BYTES) + pr_dst0;
        const int64_t byte0 = (int64_t)j * SPAN;                          // first code byte of the stage within a row
        const bool valid = kbyte0 + byte0 + pr_pc * 16 < row_bytes;       // K tail: zero-fill instead of reading
        const unsigned char* src = pr_src0 + (valid ? byte0 : 0);
#pragma unroll
        for (int t = 0; t < TC_M / RSTEP; ++t) {
          int r = pr_r0 + t * RSTEP;
          r = r < rmax ? r : rmax;                                        // rows past the matrix re-read its last row
          tc_cp_async16(dst + (uint32_t)(t * RSTEP * SPAN), src + (int64_t)r * row_bytes, valid ? 16u : 0u);
        }
      }
      tc_cp_async_commit();                                 // one group per stage index, empty past the end
    };

    // ---- conversion: item i = tid + W t of a chunk is row (i & 127), 16-byte piece (i >> 7) of the chunk's raw bytes
    const int cv_r = tid & 127, cv_q = tid >> 7, cv_s = cv_r & 7;
    const uint32_t cv_src = (uint32_t)(cv_r * SPAN);
    const uint32_t cv_dst = (uint32_t)(cv_r * 128);

    // ---- read-out of chunk cc: readout_begin waits for the chunk's MMAs and starts the loads of its (up to) two
    //      accumulators; readout_end waits for the loads and adds  d[row][block] * accumulator  into acc.
    uint32_t r0[NCOL], r1[NCOL];
    auto readout_begin = [&](int cc) {
      const int set = cc % D;
      if (alive && !tc_mbar_wait(bar_mma + 8u * set, (uint32_t)((cc / D) & 1))) {
        alive = false;
        if (lane == 0) *p.err_flag = 1;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = t_lane + (uint32_t)(set * 2 * ACC_STRIDE);
      tc_tmem_ld<NCOL>(taddr, r0);
      if (2 * cc + 1 < n_blocks) tc_tmem_ld<NCOL>(taddr + ACC_STRIDE, r1);
    };
    auto readout_end = [&](int cc) {
      if ((cc & 3) == 0) {
        sc_cur = sc_next;
        if (cc + 4 < n_chunks) sc_next = srow[(cc >> 2) + 1];
      }
      const int sel = cc & 3;
      const uint32_t dw = sel == 0 ? sc_cur.x : (sel == 1 ? sc_cur.y : (sel == 2 ? sc_cur.z : sc_cur.w));
      const float d0 = __half2float(__ushort_as_half((unsigned short)(dw & 0xFFFF)));
      const float d1 = __half2float(__ushort_as_half((unsigned short)(dw >> 16)));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const f32x2_t dd0 = pack2(d0, d0), dd1 = pack2(d1, d1);
#pragma unroll
      for (int j = 0; j < NCOL / 2; ++j) acc2[j] = fma2(dd0, pack2(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1])), acc2[j]);
      if (2 * cc + 1 < n_blocks) {
#pragma unroll
        for (int j = 0; j < NCOL / 2; ++j) acc2[j] = fma2(dd1, pack2(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1])), acc2[j]);
      }
      // orders the loads above before the arrival that lets an MMA warp overwrite these accumulators
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    for (int j = 0; j < TC_RAW_STAGES; ++j) issue_raw(j);
    pdl_wait();                                             // (weights are constants: their first stages are already on the way)
    // this thread's copies of stage 0 have landed; after the barrier, every worker's
    tc_cp_async_wait(TC_RAW_STAGES - 1);
    asm volatile("bar.sync 1, %0;" ::"n"(W) : "memory");

    int c = 0;
    for (int rs = 0; rs < n_stages; ++rs) {
      const uint32_t raw = raw_st + (uint32_t)((rs & (TC_RAW_STAGES - 1)) * RAW_BYTES) + cv_src;
#pragma unroll
      for (int u = 0; u < SUB; ++u) {
        if (c < n_chunks) {
          const int set = c % D;
          // (b) raw codes -> fp16 integers in the swizzled A-tile layout. The tile was last read by the MMAs of
          //     chunk c-D, whose completion this thread awaited in an earlier iteration. Loads first, so that
          //     their latency overlaps.
          const uint32_t a_t = a_st + (uint32_t)(set * TC_A_BYTES) + cv_dst;
          if (TYPE == CAI_TYPE_Q8_0) {
            constexpr uint32_t BIAS = 0x64806480u;          // fp16 1152 = 1024 + 128: stored codes are q + 128
            constexpr int ITEMS = 512 / W;
            uint4 w[ITEMS];
#pragma unroll
            for (int t = 0; t < ITEMS; ++t) w[t] = tc_lds128(raw + (uint32_t)((((u * 4 + cv_q + (W / 128) * t) ^ cv_s)) << 4));
#pragma unroll
            for (int t = 0; t < ITEMS; ++t) {               // row fastest: 8 consecutive threads touch 8 distinct bank groups
              const int q = cv_q + (W / 128) * t;
              tc_sts128(a_t + (uint32_t)(((2 * q) ^ cv_s) << 4), bytes_to_half2(w[t].x, 0x4140, BIAS), bytes_to_half2(w[t].x, 0x4342, BIAS),
                        bytes_to_half2(w[t].y, 0x4140, BIAS), bytes_to_half2(w[t].y, 0x4342, BIAS));
              tc_sts128(a_t + (uint32_t)(((2 * q + 1) ^ cv_s) << 4), bytes_to_half2(w[t].z, 0x4140, BIAS), bytes_to_half2(w[t].z, 0x4342, BIAS),
                        bytes_to_half2(w[t].w, 0x4140, BIAS), bytes_to_half2(w[t].w, 0x4342, BIAS));
            }
          } else if (tid < 256) {                           // 256 blocks of 32 nibble codes per chunk: one per thread
            constexpr uint32_t BIAS = 0x64086408u;          // fp16 1032 = 1024 + 8
            const int blk = cv_q;
            const uint4 w = tc_lds128(raw + (uint32_t)((((u * 2 + blk) ^ cv_s)) << 4));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { lo[i] = ww[i] & 0x0F0F0F0Fu; hi[i] = (ww[i] >> 4) & 0x0F0F0F0Fu; }
            // byte e of the block: element e in the low nibble, element e + 16 in the high nibble
            const int j0 = 4 * blk;
            tc_sts128(a_t + (uint32_t)(((j0 + 0) ^ cv_s) << 4), bytes_to_half2(lo[0], 0x4140, BIAS), bytes_to_half2(lo[0], 0x4342, BIAS),
                      bytes_to_half2(lo[1], 0x4140, BIAS), bytes_to_half2(lo[1], 0x4342, BIAS));
            tc_sts128(a_t + (uint32_t)(((j0 + 1) ^ cv_s) << 4), bytes_to_half2(lo[2], 0x4140, BIAS), bytes_to_half2(lo[2], 0x4342, BIAS),
                      bytes_to_half2(lo[3], 0x4140, BIAS), bytes_to_half2(lo[3], 0x4342, BIAS));
            tc_sts128(a_t + (uint32_t)(((j0 + 2) ^ cv_s) << 4), bytes_to_half2(hi[0], 0x4140, BIAS), bytes_to_half2(hi[0], 0x4342, BIAS),
                      bytes_to_half2(hi[1], 0x4140, BIAS), bytes_to_half2(hi[1], 0x4342, BIAS));
            tc_sts128(a_t + (uint32_t)(((j0 + 3) ^ cv_s) << 4), bytes_to_half2(hi[2], 0x4140, BIAS), bytes_to_half2(hi[2], 0x4342, BIAS),
                      bytes_to_half2(hi[3], 0x4140, BIAS), bytes_to_half2(hi[3], 0x4342, BIAS));
          }
          // (c) make the stores visible to the tensor-core (async) proxy and tell the chunk's MMA warp: the tile is
          //     ready, and this thread is done with the accumulators of chunk c-D (read out in the previous iteration)
          //     One arrival per warp: 256 separate arrivals on one barrier word serialize.
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_a + 8u * set) : "memory");
          // (d) fold chunk c-(D-1) into the registers: its MMAs were issued D-1 iterations ago. (Starting the
          //     tensor-memory loads before the conversion, to hide their latency, measured no gain, and registers
          //     with such a load in flight must not be touched, not even by a spill, until the wait.)
          if (c >= D - 1) {
            readout_begin(c - (D - 1));
            readout_end(c - (D - 1));
          }
          ++c;
        }
      }
      // (e) one barrier per stage: this thread's copies of the next stage have landed and it has converted this
      //     stage's last chunk; after the barrier that holds for every worker, so the slot can be refilled
      tc_cp_async_wait(0);
      asm volatile("bar.sync 1, %0;" ::"n"(W) : "memory");
      issue_raw(rs + TC_RAW_STAGES);
    }
    for (int cc = (n_chunks >= D - 1 ? n_chunks - (D - 1) : 0); cc < n_chunks; ++cc) { readout_begin(cc); readout_end(cc); }
    tc_cp_async_wait(0);

    // ---- epilogue: thread = weight row, acc[j] = batch column cg * NCOL + j ----
    float acc[NCOL];
#pragma unroll
    for (int j = 0; j < NCOL / 2; ++j) asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[2 * j]), "=f"(acc[2 * j + 1]) : "l"(acc2[j]));
    if (row_ok && p.ksplit > 1) {
      float* part = p.part + (size_t)blockIdx.y * (size_t)p.batch * (size_t)p.n + my_row;
#pragma unroll
      for (int j = 0; j < NCOL; ++j) {
        const int b = cg * NCOL + j;
        if (b < p.batch) part[(size_t)b * (size_t)p.n] = acc[j] * unscale[b];
      }
    } else if (row_ok) {
      const float bias = p.bias ? p.bias[my_row] : 0.f;
#pragma unroll
      for (int j = 0; j < NCOL; ++j) {
        const int b = cg * NCOL + j;
        const int64_t orow = out_rows ? (int64_t)out_rows[b] : (int64_t)b;     // grouped: scatter to the pair's row
        if (out_rows ? (orow >= 0) : (b < p.batch)) {
          float v = fmaf(acc[j], unscale[b], bias);
          v = apply_act(v, p.act);
          if (p.epi == EPI_RESID) v += p.resid[orow * p.ldy + my_row];
          p.y[orow * p.ldy + my_row] = v;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)Plan::TMEM_COLS) : "memory");
}

template <int TYPE, int NB>
cudaError_t tc_launch(cai_ctx* ctx, const TcParams& p, int grid, int tiles = 1) {
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TYPE, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcPlan<NB>::SMEM);
  if (e == cudaSuccess)
    e = pdl_launch(ctx, gemm_tc_kernel<TYPE, NB>, dim3((unsigned)grid, (unsigned)p.ksplit, (unsigned)tiles), dim3(TcPlan<NB>::THREADS), (size_t)TcPlan<NB>::SMEM, p);
  return e;
}

// y[b][row] = act(sum over splits of part[s][b][row] + bias) (+ residual), splits added in index order
__global__ void tc_reduce_kernel(const float* __restrict__ part, int ksplit, int batch, int64_t n, const float* __restrict__ bias,
                                 const float* __restrict__ resid, float* __restrict__ y, int64_t ldy, int act, int epi) {
  pdl_trigger();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)batch * n) return;
  const int64_t b = i / n, row = i - b * n;
  float v = 0.f;
  for (int s = 0; s < ksplit; ++s) v += part[((size_t)s * batch + b) * n + row];
  if (bias) v += bias[row];
  v = apply_act(v, act);
  if (epi == EPI_RESID) v += resid[b * ldy + row];
  y[b * ldy + row] = v;
}

}  // namespace

// Grows the buffer that holds the split activations. Sessions size it when they are created, so a step
// that is being captured into a graph never allocates. An outgrown buffer is kept until the context is
// destroyed, because a graph captured earlier may still name it; sizes at least double, so few are kept.
// Grows the buffer that holds the split activations. Sessions size it when they are created, so a step
// that is being captured into a graph never allocates. An outgrown buffer is kept until the context is
// destroyed, because a graph captured earlier may still name it; sizes at least double, so few are kept.
constexpr size_t TC_PART_ROWS = 12800;   // K is split only for matrices of at most this many rows ...
constexpr int TC_MAX_KSPLIT = 16;        // ... into at most this many ranges
static size_t tc_xp_bytes_for(int64_t k, int nb) { return ((256 + (size_t)((k + TC_KC - 1) / TC_KC) * 2 * (size_t)nb * 128) + 255) & ~(size_t)255; }

int gemm_tc_reserve(cai_ctx* ctx, int64_t k, int batch) {
  const int nb = batch <= 16 ? 16 : (batch <= 32 ? 32 : 64);
  // 64 row factors and two limbs per chunk, then the partial sums of a K-split call
  size_t need = tc_xp_bytes_for(k, nb) + (size_t)TC_MAX_KSPLIT * nb * TC_PART_ROWS * 4;
  if (need <= ctx->tc_xp_bytes) return CAI_OK;
  if (need < 2 * ctx->tc_xp_bytes) need = 2 * ctx->tc_xp_bytes;
  if (ctx->tc_xp) {
    if (ctx->tc_xp_n_retired >= 32) return cai_fail(ctx, CAI_ERR_OOM, "tensor-core GEMM: activation buffer regrown too often");
    ctx->tc_xp_retired[ctx->tc_xp_n_retired++] = ctx->tc_xp;
    ctx->tc_xp = nullptr;
    ctx->tc_xp_bytes = 0;
  }
  CAI_CUDA(ctx, cudaMalloc(&ctx->tc_xp, need));
  ctx->tc_xp_bytes = need;
  return CAI_OK;
}

// Launches the tensor-core GEMM, or returns CAI_ERR_UNSUPPORTED (no message) when the call is outside
// what it covers: batches of 1..64 rows, plain or residual epilogue, Q8_0 / Q4_0 weights, no expert indexing.
// (Which batches are worth sending here is the caller's policy.)
int gemm_tc_launch(cai_ctx* ctx, const GemvParams& g, int type) {
  if (!ctx->err_flag || g.expert_ids || g.batch < 1 || g.batch > 64) return CAI_ERR_UNSUPPORTED;
  if (g.epi != EPI_STORE && g.epi != EPI_RESID) return CAI_ERR_UNSUPPORTED;
  if (g.row_scale) return CAI_ERR_UNSUPPORTED;
  if (((uintptr_t)g.x % 16) || (g.ldx % 4) || ((uintptr_t)g.codes % 16)) return CAI_ERR_UNSUPPORTED;
  if (g.norm_gain && ((uintptr_t)g.norm_gain % 16)) return CAI_ERR_UNSUPPORTED;
  CAI_TRY(gemm_tc_reserve(ctx, g.k, g.batch));
  const int nb = g.batch <= 16 ? 16 : (g.batch <= 32 ? 32 : 64);
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.codes = (const unsigned char*)g.codes; p.scales = g.scales; p.bias = g.bias;
  p.row_unscale = (const float*)ctx->tc_xp; p.xp = (const unsigned char*)ctx->tc_xp + 256;
  p.y = g.y; p.ldy = g.ldy; p.resid = g.resid;
  p.n = g.n; p.k = g.k; p.sstride = g.sstride; p.batch = g.batch; p.act = g.act; p.epi = g.epi;
  p.err_flag = ctx->err_flag;
  const int n_chunks = (int)((g.k + TC_KC - 1) / TC_KC);
  {
    const int threads = g.k >= 2048 ? 512 : 256;
    pdl_launch(ctx, tc_split_x_kernel, dim3(nb), dim3(threads), 0, g.x, g.ldx, g.batch, nb, g.k, n_chunks, 2, g.norm_gain, g.norm_eps,
               (unsigned char*)ctx->tc_xp + 256, (float*)ctx->tc_xp, (const int32_t*)nullptr, 1, (size_t)0);
    CAI_LAUNCHED(ctx);
  }
  const int grid = (int)((g.n + TC_M - 1) / TC_M);
  // Fewer row tiles than SMs: split K over blockIdx.y so that the launch fills the machine (two CTAs per SM), each
  // range a multiple of 8 chunks. (Matrices with 75..148 row tiles were left whole at first; splitting them in two
  // measured 4 % on the TinyLlama step although it adds the launch that sums the ranges.)
  p.ksplit = 1;
  p.chunks_per_split = n_chunks;
  // (ranges of 8 chunks, the shortest the stage geometry allows, measured 8 % faster than 16 on the 2048-wide matrices
  // of the TinyLlama shape: those launches are latency chains, and a CTA's chain is as long as its K range)
  const int min_cps = env_int("CAI_TC_MINCPS", 8);
  if (grid <= ctx->sm_count && (size_t)g.n <= TC_PART_ROWS && n_chunks >= 2 * min_cps) {
    int ks = (2 * ctx->sm_count) / grid;
    if (ks > TC_MAX_KSPLIT) ks = TC_MAX_KSPLIT;
    ks = env_int("CAI_TC_KSPLIT", ks);
    if (ks < 1) ks = 1;
    if (ks > TC_MAX_KSPLIT) ks = TC_MAX_KSPLIT;
    int cps = (n_chunks + ks - 1) / ks;
    if (cps < min_cps) cps = min_cps;
    cps = (cps + 7) & ~7;
    p.chunks_per_split = cps;
    p.ksplit = (n_chunks + cps - 1) / cps;
    p.part = (float*)((unsigned char*)ctx->tc_xp + tc_xp_bytes_for(g.k, nb));
  }
  cudaError_t e;
  if (type == CAI_TYPE_Q8_0)
    e = nb == 16 ? tc_launch<CAI_TYPE_Q8_0, 16>(ctx, p, grid) : (nb == 32 ? tc_launch<CAI_TYPE_Q8_0, 32>(ctx, p, grid) : tc_launch<CAI_TYPE_Q8_0, 64>(ctx, p, grid));
  else
    e = nb == 16 ? tc_launch<CAI_TYPE_Q4_0, 16>(ctx, p, grid) : (nb == 32 ? tc_launch<CAI_TYPE_Q4_0, 32>(ctx, p, grid) : tc_launch<CAI_TYPE_Q4_0, 64>(ctx, p, grid));
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "gemm_tc smem attribute -> %s", cudaGetErrorString(e));
  CAI_LAUNCHED(ctx);
  if (p.ksplit > 1) {
    const int64_t total = (int64_t)g.batch * g.n;
    pdl_launch(ctx, tc_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (const float*)p.part, p.ksplit, g.batch, g.n, g.bias, g.resid, g.y, g.ldy, g.act, g.epi);
    CAI_LAUNCHED(ctx);
  }
  return CAI_OK;
}

// Bytes of split activations one 16-row tile of a grouped call needs for rows of k values.
size_t gemm_tc_group_tile_bytes(int64_t k) { return (size_t)((k + TC_KC - 1) / TC_KC) * 2 * 16 * 128; }

// Grouped tensor-core GEMM for a mixture-of-experts layer: n_tiles tiles of up to 16 (token, expert) pairs, all pairs
// of a tile routed to the same expert (op_moe_group builds the lists). One launch of the activation split and one of
// the GEMM cover every tile, so an expert's weights are streamed once per 16 pairs instead of once per pair.
// y row of pair p = p; x row of pair p = p / x_row_div. Plain epilogue.
int gemm_tc_launch_grouped(cai_ctx* ctx, int type, const void* const* bank_codes, const __half* const* bank_scales, int64_t n, int64_t k,
                           int64_t sstride, const float* x, int64_t ldx, int x_row_div, float* y, int64_t ldy,
                           const int32_t* tile_expert, const int32_t* tile_pairs, int n_tiles, void* xp_tiles, float* unscale_tiles) {
  if (!ctx->err_flag) return cai_fail(ctx, CAI_ERR_STATE, "grouped GEMM: context without error word");
  if (type != CAI_TYPE_Q8_0 && type != CAI_TYPE_Q4_0) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "grouped GEMM: Q8_0 / Q4_0 experts only");
  if (((uintptr_t)x % 16) || (ldx % 4) || (k % 32)) return cai_fail(ctx, CAI_ERR_INVALID, "grouped GEMM: activations must be 16-byte aligned, K a multiple of 32");
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.y = y; p.ldy = ldy; p.n = n; p.k = k; p.sstride = sstride; p.batch = 16; p.act = CAI_ACT_NONE; p.epi = EPI_STORE;
  p.err_flag = ctx->err_flag;
  p.xp = (const unsigned char*)xp_tiles; p.row_unscale = unscale_tiles;
  p.tile_expert = tile_expert; p.tile_pairs = tile_pairs; p.bank_codes = bank_codes; p.bank_scales = bank_scales;
  p.xp_tile_bytes = gemm_tc_group_tile_bytes(k);
  const int n_chunks = (int)((k + TC_KC - 1) / TC_KC);
  p.ksplit = 1; p.chunks_per_split = n_chunks;
  pdl_launch(ctx, tc_split_x_kernel, dim3(16, (unsigned)n_tiles), dim3(k >= 2048 ? 512 : 256), 0, x, ldx, 16, 16, k, n_chunks, 2, (const float*)nullptr, 0.f,
             (unsigned char*)xp_tiles, unscale_tiles, tile_pairs, x_row_div, p.xp_tile_bytes);
  CAI_LAUNCHED(ctx);
  const int grid = (int)((n + TC_M - 1) / TC_M);
  const cudaError_t e = (type == CAI_TYPE_Q8_0) ? tc_launch<CAI_TYPE_Q8_0, 16>(ctx, p, grid, n_tiles) : tc_launch<CAI_TYPE_Q4_0, 16>(ctx, p, grid, n_tiles);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "gemm_tc smem attribute -> %s", cudaGetErrorString(e));
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
