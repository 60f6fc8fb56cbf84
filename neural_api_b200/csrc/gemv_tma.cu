// Stream-K dequant-fused GEMV for Q8_0 / Q4_0 with bulk-copy (TMA) staging.
//
// Work unit = (row group of 32 rows, K tile of 1024 codes): 34 KB of codes+scales for
// Q8_0. All units of the matrix, K tile fastest, are cut into equal contiguous ranges,
// one per persistent CTA (2 CTAs per SM), so every SM streams the same number of bytes
// whatever the shape: small-N / large-K matrices split K across CTAs, large-N matrices
// give each CTA several row groups. A producer warp moves each unit into a ring of
// shared-memory stages with cp.async.bulk (one copy per row for codes, one for scales,
// one per activation row for the x tile), completion on an mbarrier; 8 consumer warps
// (4 rows each) read the stage, convert codes exactly to fp32 and accumulate with
// packed fp32x2 FMAs; a second mbarrier hands the stage back. The global->shared
// traffic never passes through registers or the L1 load path, and S stages per CTA
// are in flight per SM.
//
// A row group whose K range is shared by several CTAs is finished by the LAST of them
// to arrive (atomic ticket, no waiting): every CTA leaves its partial sums in a scratch
// slot, the last one adds the slots in CTA order (a fixed order: results do not depend
// on timing) and runs the epilogue. Tickets reset themselves.
//
// Every wait on an mbarrier is bounded; if one runs out the kernel raises the context's
// error word and leaves, it never spins forever.
#include "gemv_common.cuh"

namespace {

constexpr int TMA_R = 32;             // rows per group (8 consumer warps x 4 rows)
constexpr int TMA_CONSUMER_WARPS = 8;
constexpr int TMA_RPW = TMA_R / TMA_CONSUMER_WARPS;
constexpr int TMA_THREADS = (TMA_CONSUMER_WARPS + 1) * 32;
constexpr uint32_t TMA_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
  return ok != 0;
}
// Bounded wait: false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < TMA_SPIN_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// global -> shared bulk copy (TMA, untiled), bytes and both addresses multiples of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void consumer_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(TMA_CONSUMER_WARPS * 32) : "memory"); }

// One stage holds 1024 codes per row: two 16-byte chunks per lane for Q8_0, one for Q4_0.
// (Measured: 512-code stages with four stages per CTA were 40 % slower - the per-row bulk copies
// get too small - so the stage stays large and the ring short.)
template <int TYPE, int NB>
struct StageLayout {
  static constexpr int KT = 1024;                                        // codes per row per stage
  static constexpr int STAGES = 2;
  static constexpr int CODE_B = (TYPE == CAI_TYPE_Q8_0) ? KT : KT / 2;   // code bytes per row
  static constexpr int SC_B = (KT / 16 + 15) / 16 * 16;                  // scale bytes per row, 16-byte multiple
  static constexpr int ROW_B = CODE_B + SC_B;
  static constexpr int X_OFF = TMA_R * ROW_B;
  static constexpr int STAGE_B = X_OFF + NB * KT * 4;
};

struct TmaExtra {
  float* scratch;        // [ctas][2][TMA_R][NB] partial sums of split row groups
  int* tickets;          // [groups] arrival counters, zero between launches
  int n_groups;
  int n_tiles;           // K tiles per row group
  int units_per_cta;
};

template <int TYPE, int NB>
__global__ void __launch_bounds__(TMA_THREADS, 2) gemv_tma_kernel(const GemvParams p, const TmaExtra e) {
  using L = StageLayout<TYPE, NB>;
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TMA_KT = L::KT;
  constexpr int TMA_STAGES = L::STAGES;
  __shared__ __align__(8) uint64_t bars[2 * TMA_STAGES];     // full[S], empty[S]
  __shared__ int s_last;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int T = e.n_tiles;
  const int64_t U = (int64_t)e.n_groups * T;
  const int64_t u_begin = (int64_t)blockIdx.x * e.units_per_cta;
  int64_t u_end = u_begin + e.units_per_cta;
  if (u_end > U) u_end = U;
  if (u_begin >= u_end) return;

  const uint32_t bar0 = smem_u32(bars);
  if (threadIdx.x == 0) {
    for (int s = 0; s < TMA_STAGES; ++s) {
      mbar_init(bar0 + 8 * s, 1);                                  // full: the producer's arrive + bytes
      mbar_init(bar0 + 8 * (TMA_STAGES + s), TMA_CONSUMER_WARPS);  // empty: one arrive per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  const int64_t K = p.k;
  const int64_t half_n = p.n >> 1;
  const bool swiglu = (p.epi == EPI_SWIGLU);
  const int64_t units_per_group = swiglu ? (TMA_R / 2) : TMA_R;     // output units per row group

  if (warp == TMA_CONSUMER_WARPS) {
    // ------------------------------ producer ------------------------------
    const char* codes = (const char*)p.codes;
    const int64_t row_bytes = (TYPE == CAI_TYPE_Q8_0) ? K : (K >> 1);
    int64_t cur_g = -1;
    int64_t row = 0;
    uint32_t it = 0;
    bool alive = true;
    for (int64_t u = u_begin; u < u_end; ++u, ++it) {
      const int64_t g = u / T;
      const int t = (int)(u - g * T);
      const int slot = (int)(it % TMA_STAGES);
      if (g != cur_g) {
        cur_g = g;
        // row slot `lane` of the group -> weight row (clamped: surplus rows are loaded but never stored)
        if (swiglu) {
          int64_t j = g * units_per_group + (lane >> 1);
          if (j >= half_n) j = half_n - 1;
          row = (lane & 1) ? half_n + j : j;
        } else {
          row = g * TMA_R + lane;
          if (row >= p.n) row = p.n - 1;
        }
      }
      // After a wait has run out nothing is waited for any more: the loop still runs to its end so that
      // every barrier keeps its arrival count (the results are garbage and the error word says so).
      if (alive && !mbar_wait(bar0 + 8 * (TMA_STAGES + slot), ((it / TMA_STAGES) & 1) ^ 1)) {
        alive = false;
        if (lane == 0) *p.err_flag = 1;
      }
      const int64_t k0 = (int64_t)t * TMA_KT;
      const int len = (int)((K - k0 < TMA_KT) ? (K - k0) : TMA_KT);
      const uint32_t cb = (TYPE == CAI_TYPE_Q8_0) ? (uint32_t)len : (uint32_t)(len >> 1);
      const uint32_t sb = ((uint32_t)(len >> 4) + 15u) & ~15u;
      const uint32_t full = bar0 + 8 * slot;
      if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)TMA_R * (cb + sb) + (uint32_t)NB * (uint32_t)len * 4u);
      __syncwarp();
      const uint32_t stage = smem_u32(smem) + (uint32_t)slot * L::STAGE_B;
      bulk_g2s(stage + lane * L::ROW_B, codes + row * row_bytes + ((TYPE == CAI_TYPE_Q8_0) ? k0 : (k0 >> 1)), cb, full);
      bulk_g2s(stage + lane * L::ROW_B + L::CODE_B, p.scales + row * p.sstride + (k0 >> 5), sb, full);
      if (lane < NB) {
        const int bb = (lane < p.batch) ? lane : 0;
        bulk_g2s(stage + L::X_OFF + lane * (TMA_KT * 4), p.x + (int64_t)bb * p.ldx + k0, (uint32_t)len * 4u, full);
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  f32x2_t acc2[TMA_RPW][NB];
#pragma unroll
  for (int r = 0; r < TMA_RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc2[r][b] = 0ull;

  uint32_t it = 0;
  bool alive = true;
  for (int64_t u = u_begin; u < u_end; ++u, ++it) {
    const int64_t g = u / T;
    const int t = (int)(u - g * T);
    const int slot = (int)(it % TMA_STAGES);
    if (alive && !mbar_wait(bar0 + 8 * slot, (it / TMA_STAGES) & 1)) {
      alive = false;
      if (lane == 0) *p.err_flag = 1;
    }
    const int64_t k0 = (int64_t)t * TMA_KT;
    const int len = (int)((K - k0 < TMA_KT) ? (K - k0) : TMA_KT);
    const unsigned char* stage = smem + (size_t)slot * L::STAGE_B;
    const float* xt = (const float*)(stage + L::X_OFF);
    constexpr int CHUNK = (TYPE == CAI_TYPE_Q8_0) ? 16 : 32;          // codes per 16-byte lane chunk
#pragma unroll
    for (int kk = 0; kk < TMA_KT; kk += 32 * CHUNK) {
      const int kc = kk + lane * CHUNK;                                // first code of this lane's chunk
      if (kc < len) {
        int4 wv[TMA_RPW];
        uint32_t sv[TMA_RPW];
#pragma unroll
        for (int r = 0; r < TMA_RPW; ++r) {
          const unsigned char* rowp = stage + (warp * TMA_RPW + r) * L::ROW_B;
          wv[r] = *(const int4*)(rowp + ((TYPE == CAI_TYPE_Q8_0) ? kc : (kc >> 1)));
          sv[r] = *(const unsigned short*)(rowp + L::CODE_B + (kc >> 5) * 2);
        }
        f32x2_t part[TMA_RPW][NB];
#pragma unroll
        for (int r = 0; r < TMA_RPW; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b) part[r][b] = 0ull;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (TYPE == CAI_TYPE_Q8_0) {
            float4 xv[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) xv[b] = *(const float4*)(xt + b * TMA_KT + kc + 4 * i);
#pragma unroll
            for (int r = 0; r < TMA_RPW; ++r) {
              const uint32_t w = ((const uint32_t*)&wv[r])[i];
#pragma unroll
              for (int b = 0; b < NB; ++b) part[r][b] = q8_word_fma(w, xv[b], part[r][b]);
            }
          } else {
            float4 xlo[NB], xhi[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              xlo[b] = *(const float4*)(xt + b * TMA_KT + kc + 4 * i);
              xhi[b] = *(const float4*)(xt + b * TMA_KT + kc + 16 + 4 * i);
            }
#pragma unroll
            for (int r = 0; r < TMA_RPW; ++r) {
              const uint32_t w = ((const uint32_t*)&wv[r])[i];
#pragma unroll
              for (int b = 0; b < NB; ++b) part[r][b] = q4_word_fma(w, xlo[b], xhi[b], part[r][b]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < TMA_RPW; ++r) {
          const float d = half_bits_to_float(sv[r]);
          const f32x2_t d2 = pack2(d, d);
#pragma unroll
          for (int b = 0; b < NB; ++b) acc2[r][b] = fma2(d2, part[r][b], acc2[r][b]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar0 + 8 * (TMA_STAGES + slot));    // stage may be refilled

    const bool group_end = (t == T - 1) || (u == u_end - 1);
    if (!group_end) continue;

    float acc[TMA_RPW][NB];
#pragma unroll
    for (int r = 0; r < TMA_RPW; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) { acc[r][b] = warp_sum(sum2(acc2[r][b])); acc2[r][b] = 0ull; }

    const int64_t ug0 = g * T;                                       // first unit of this row group
    const bool whole = (u_begin <= ug0) && (ug0 + T <= u_end);
    bool finish = whole;
    if (!whole) {
      // leave this CTA's partial sums in its scratch slot and take a ticket
      const int64_t q = e.units_per_cta;
      const int c_first = (int)(ug0 / q), c_last = (int)((ug0 + T - 1) / q);
      const int parts = c_last - c_first + 1;
      const int which = (ug0 >= u_begin) ? 1 : 0;                    // 1: the group starts inside this CTA's range
      float* mine = e.scratch + (((size_t)blockIdx.x * 2 + which) * TMA_R + (size_t)warp * TMA_RPW) * NB;
      if (lane < TMA_RPW * NB) {
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < TMA_RPW; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b)
            if (lane == r * NB + b) v = acc[r][b];
        __stcg(mine + lane, v);
      }
      __threadfence();
      consumer_bar_sync();
      if (threadIdx.x == 0) {
        const int old = atomicAdd(e.tickets + g, 1);
        s_last = (old == parts - 1) ? 1 : 0;
        if (old == parts - 1) e.tickets[g] = 0;                      // ready for the next launch
      }
      consumer_bar_sync();
      finish = (s_last != 0);
      if (finish) {
        __threadfence();
        float v = 0.f;
        if (lane < TMA_RPW * NB) {
          for (int i = 0; i < parts; ++i) {                           // fixed order: CTA index
            const int c = c_first + i;
            const int w2 = (ug0 >= (int64_t)c * q) ? 1 : 0;
            v += __ldcg(e.scratch + (((size_t)c * 2 + w2) * TMA_R + (size_t)warp * TMA_RPW) * NB + lane);
          }
        }
#pragma unroll
        for (int r = 0; r < TMA_RPW; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b) acc[r][b] = __shfl_sync(0xffffffffu, v, r * NB + b);
      }
      consumer_bar_sync();   // s_last is reused by the next split group
    }
    if (finish) {
      const int64_t unit0 = g * units_per_group + (int64_t)warp * (swiglu ? TMA_RPW / 2 : TMA_RPW);
      gemv_epilogue<NB, TMA_RPW>(p, acc, unit0, 0, 0, p.bias);
    }
  }
}

template <int TYPE, int NB>
int launch_tma(cai_ctx* ctx, const GemvParams& p, const TmaExtra& e, int ctas) {
  using L = StageLayout<TYPE, NB>;
  const size_t smem = (size_t)L::STAGES * L::STAGE_B;
  cudaError_t err = cudaFuncSetAttribute(gemv_tma_kernel<TYPE, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "gemv_tma smem attribute -> %s", cudaGetErrorString(err));
  gemv_tma_kernel<TYPE, NB><<<ctas, TMA_THREADS, smem, ctx->stream>>>(p, e);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

}  // namespace

// Returns CAI_OK after launching, or CAI_ERR_UNSUPPORTED (without an error message) when the shape is
// outside what this kernel covers and the caller should use the register-staged kernel.
int gemv_tma_launch(cai_ctx* ctx, GemvParams p, int type, int nb) {
  if (!ctx->gemv_scratch || !ctx->gemv_tickets || !ctx->err_flag) return CAI_ERR_UNSUPPORTED;
  if (p.expert_ids || nb > 4 || p.batch > nb) return CAI_ERR_UNSUPPORTED;
  if (((uintptr_t)p.x % 16) || (p.ldx % 4)) return CAI_ERR_UNSUPPORTED;
  const bool swiglu = (p.epi == EPI_SWIGLU);
  const int64_t units = swiglu ? p.n / 2 : p.n;
  const int64_t upg = swiglu ? TMA_R / 2 : TMA_R;
  const int64_t groups = (units + upg - 1) / upg;
  if (groups > ctx->gemv_ticket_cap) return CAI_ERR_UNSUPPORTED;
  TmaExtra e;
  e.scratch = ctx->gemv_scratch;
  e.tickets = ctx->gemv_tickets;
  e.n_groups = (int)groups;
  const int kt = 1024;
  e.n_tiles = (int)((p.k + kt - 1) / kt);
  const int64_t U = groups * e.n_tiles;
  int ctas = ctx->gemv_scratch_ctas;                 // 2 per SM
  if (U < ctas) ctas = (int)U;
  e.units_per_cta = (int)((U + ctas - 1) / ctas);
  ctas = (int)((U + e.units_per_cta - 1) / e.units_per_cta);
  p.err_flag = ctx->err_flag;
  if (type == CAI_TYPE_Q8_0) {
    if (nb == 1) return launch_tma<CAI_TYPE_Q8_0, 1>(ctx, p, e, ctas);
    if (nb == 2) return launch_tma<CAI_TYPE_Q8_0, 2>(ctx, p, e, ctas);
    return launch_tma<CAI_TYPE_Q8_0, 4>(ctx, p, e, ctas);
  }
  if (nb == 1) return launch_tma<CAI_TYPE_Q4_0, 1>(ctx, p, e, ctas);
  if (nb == 2) return launch_tma<CAI_TYPE_Q4_0, 2>(ctx, p, e, ctas);
  return launch_tma<CAI_TYPE_Q4_0, 4>(ctx, p, e, ctas);
}
