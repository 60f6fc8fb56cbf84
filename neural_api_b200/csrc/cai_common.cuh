// Internal declarations shared by the translation units of libcai_cuda.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>
#include <vector>
#include <string>
#include "../../include/cai_cuda.h"

#define CAI_QK 32
#define CAI_Q8_0_BLOCK_BYTES 34
#define CAI_Q4_0_BLOCK_BYTES 18

struct cai_comm_state;  // comm.cu

struct cai_ctx {
  int device;
  int sm_count;
  size_t total_mem;
  cudaStream_t stream;
  cudaEvent_t ev_begin, ev_end;
  char err[1024];
  int64_t launches;          // kernels launched by this library on this context
  void* l2_flush_buf;        // lazily allocated, > L2 size
  size_t l2_flush_bytes;
  void* staging_dev;         // upload staging (device)
  size_t staging_bytes;
  void* staging_pinned;      // upload staging (pinned host)
  cai_comm_state* comm;      // NULL until cai_comm_init
  int* err_flag;             // pinned, device-visible, 4 words: [0] raised by a kernel whose bounded wait ran out (1), that
                             // refused a cache length outside the cache (2), that met an unusable router row (3) or, in
                             // the checked build, that met an index outside its range (4: [1] site, [2] value, [3] bound)
  unsigned wait_limit_us;    // how long a device-side wait on another CTA or GPU may last before it gives up
  void* tc_xp;               // tensor-core GEMM: activations split into bf16 limbs, tiled (gemm_tc_reserve)
  size_t tc_xp_bytes;
  void* tc_xp_retired[32];   // outgrown buffers: captured graphs may still name them, so they live as long as the context
  int tc_xp_n_retired;
  int use_pdl;               // launch step kernels with programmatic dependent launch
  int pdl_mode;              // 1 / 0: forced on / off by the environment, -1: each session decides
  // per-launch profiling (cai_session_profile): one event after every launch
  int prof_on;
  int cur_family;            // FAM_* of the launches being enqueued
  cudaEvent_t* prof_events;
  int* prof_family;
  int prof_n, prof_cap;
};
enum { FAM_LINEAR = 0, FAM_ATTN = 1, FAM_OTHER = 2, FAM_COMM = 3, FAM_COUNT = 4 };
int cai_prof_mark(cai_ctx* ctx, int family);

int cai_fail(cai_ctx* ctx, int code, const char* fmt, ...);
int env_int(const char* name, int dflt);                    // integer environment knob, gemv.cu
int gemm_tc_reserve(cai_ctx* ctx, int64_t k, int batch);    // gemm_tc.cu
bool linear_uses_tensor_cores(const struct QWeight* w, int batch);   // gemv.cu: dispatch policy

#define CAI_CUDA(ctx, call)                                                              \
  do {                                                                                   \
    cudaError_t e__ = (call);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return cai_fail((ctx), CAI_ERR_CUDA, "%s -> %s (%s:%d)", #call,                    \
                      cudaGetErrorString(e__), __FILE__, __LINE__);                      \
  } while (0)

#define CAI_TRY(call)                  \
  do {                                 \
    int s__ = (call);                  \
    if (s__ != CAI_OK) return s__;     \
  } while (0)

// The checked build (-DCAI_CHECKED, libcai_cuda_checked.so): the same kernels, but
//   * where the ordinary build silently clamps or ignores an index that comes from device-side state (a token id, an
//     expert id), the kernel also records site, value and bound in the error words (cai_report_index), and
//   * every launch is followed by a stream synchronize and a look at the error words and at cudaGetLastError, so a
//     failure is reported by the entry point that enqueued the launch, with that launch's file and line (CUDA graphs
//     are off in this build: every step runs launch by launch).
// It is a debugging aid: nothing in it changes a result, and the ordinary build carries none of its code.
#ifdef CAI_CHECKED
#define CAI_CHECKED_BUILD 1
#else
#define CAI_CHECKED_BUILD 0
#endif
enum { CAI_SITE_EMBED_TOKEN = 1, CAI_SITE_STEP_TOKEN = 2, CAI_SITE_MOE_EXPERT = 3 };
#ifdef __CUDACC__
__device__ __forceinline__ void cai_report_index(int* err, int site, long long value, long long bound) {
#if CAI_CHECKED_BUILD
  if (err && *(volatile int*)err == 0) {
    err[1] = site; err[2] = (int)value; err[3] = (int)bound;
    __threadfence_system();
    *(volatile int*)err = 4;
  }
#endif
}
#endif
int cai_checked_after_launch(cai_ctx* ctx, const char* file, int line);   // api.cu

// Checks the launch of the kernel just enqueued and counts it.
#define CAI_LAUNCHED(ctx)                                                                \
  do {                                                                                   \
    cudaError_t e__ = cudaGetLastError();                                                \
    if (e__ != cudaSuccess)                                                              \
      return cai_fail((ctx), CAI_ERR_CUDA, "kernel launch -> %s (%s:%d)",                \
                      cudaGetErrorString(e__), __FILE__, __LINE__);                      \
    (ctx)->launches++;                                                                   \
    if ((ctx)->prof_on) cai_prof_mark((ctx), (ctx)->cur_family);                         \
    if (CAI_CHECKED_BUILD) {                                                             \
      const int c__ = cai_checked_after_launch((ctx), __FILE__, __LINE__);               \
      if (c__ != CAI_OK) return c__;                                                     \
    }                                                                                    \
  } while (0)

static inline int cai_bind(cai_ctx* ctx) {
  if (!ctx) return CAI_ERR_INVALID;
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "cudaSetDevice(%d) -> %s", ctx->device, cudaGetErrorString(e));
  return CAI_OK;
}

int cai_ensure_staging(cai_ctx* ctx, size_t bytes);
// gguf.cu: ggml types the linear kernels do not read directly (Q4_1, Q5_0, Q5_1, Q2_K .. Q6_K) are decoded on the
// device to fp32, as the reference's reader does at load time, and continue as F32 tensors
bool gguf_type_needs_decode(int type);
int gguf_decode_host(cai_ctx* ctx, int type, const void* raw_host, int64_t n_elems, float* out_host);
int gguf_upload_decoded(struct cai_model* m, cai_ctx* ctx, const char* hf_name, int type, const void* data_host, int64_t rows, int64_t cols,
                        int interleave_head_dim);

// ---------------------------------------------------------------------------
// Resident weight matrix. GGUF blocks are split into planes when uploaded so
// that rows of codes start on 16-byte boundaries (a 34-byte Q8_0 block does
// not): values stay bit-identical, d * q is formed in fp32 exactly as
// DecodeGGMLSpan does.
//   Q8_0: codes uint8 [N][K] holding q + 128 (the bias saves one logic op per word in the GEMV),      scales fp16 [N][sstride], sstride = K/32 rounded up to 8
//   Q4_0: codes uint8 [N][K/2] (the 16 nibble bytes of each block kept together),
//         scales fp16 [N][K/32]
//   F16 : codes fp16  [N][K];  F32: codes float [N][K]
// ---------------------------------------------------------------------------
struct QWeight {
  int type = -1;
  int64_t n = 0, k = 0;
  int64_t sstride = 0;         // halves between scale rows: K/32 rounded up to 8
  void* codes = nullptr;
  __half* scales = nullptr;
  float* rscale = nullptr;     // CAI_TYPE_I8ROW: one fp32 scale per row (codes are int8 + 128, like Q8_0's)
  float* bias = nullptr;       // optional, N floats
  bool owns = true;            // false for row-range views (tied LM head shard)
  bool present = false;
  size_t code_bytes() const;
  size_t scale_bytes() const;         // algorithmic (unpadded) bytes
  size_t scale_alloc_bytes() const;   // resident bytes, rows padded to sstride
  size_t bytes() const { return code_bytes() + scale_bytes(); }
  size_t row_code_bytes() const;
};

size_t cai_type_row_bytes(int type, int64_t k);   // bytes of one GGUF row of k elements
bool cai_type_supported(int type);
bool cai_type_is_kquant(int type);                 // Q4_K / Q5_K / Q6_K: resident as the file's raw super-blocks

int qweight_alloc(cai_ctx* ctx, QWeight* w, int type, int64_t n, int64_t k);
void qweight_free(QWeight* w);
QWeight qweight_rows_view(const QWeight& w, int64_t row0, int64_t nrows);
// Uploads host GGUF rows [row0,row0+nrows) x cols [col0,col0+ncols) of a [src_rows, src_cols]
// tensor into w (already allocated as nrows x ncols), optionally gathering source rows through
// the q/k interleave permutation.
int qweight_upload(cai_ctx* ctx, QWeight* w, const void* host, int64_t src_rows, int64_t src_cols,
                   int64_t row0, int64_t col0, int interleave_head_dim);
int qweight_download_blocks(cai_ctx* ctx, const QWeight* w, void* out_host, size_t cap);
int qweight_dequantize_to_dev(cai_ctx* ctx, const QWeight* w, float* out_dev);
// F32 host rows -> I8ROW storage, quantized on the device row by row (w allocated as CAI_TYPE_I8ROW); optional row gather
int qweight_upload_quantize_i8(cai_ctx* ctx, QWeight* w, const float* host, int64_t src_rows, int64_t src_cols, int64_t row0, int64_t col0,
                               int interleave_head_dim);
int quantize_rows_i8_dev(cai_ctx* ctx, const float* x_dev, int64_t rows, int64_t cols, uint8_t* codes_biased_dev, float* scales_dev);
int qweight_init_synthetic(cai_ctx* ctx, QWeight* w, uint64_t seed, uint64_t tensor_id, float std,
                           int64_t global_row0, int64_t global_col0, int64_t global_cols);
int vec_init_synthetic(cai_ctx* ctx, float* v, int64_t n, uint64_t seed, uint64_t tensor_id, float std,
                       int64_t global0, float constant /* used when std == 0 */);

// ---------------------------------------------------------------------------
// GEMV / GEMM launchers (gemv.cu, gemm_tc.cu)
// ---------------------------------------------------------------------------
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_QKV_ROPE = 3 };

struct LinearArgs {
  const QWeight* w = nullptr;
  const float* x = nullptr;      // [B][K] (ldx floats between rows)
  int64_t ldx = 0;
  float* y = nullptr;            // [B][ldy]
  int64_t ldy = 0;
  int batch = 1;
  int epilogue = EPI_STORE;
  const float* resid = nullptr;  // EPI_RESID: y = resid + W x (+bias); ld = ldy
  int act = CAI_ACT_NONE;
  int path = 0;                  // 0 auto, 1 CUDA-core GEMV only, 2 tensor-core GEMM only
  // Indexed (MoE) mode: per pair p, the weight matrix is banks[expert_ids[p]] and the
  // activation row is x + x_row[p]*ldx (x_row NULL -> p).
  const QWeight* const* bank = nullptr;  // unused (device arrays below are what kernels read)
  const void* const* bank_codes_dev = nullptr;
  const __half* const* bank_scales_dev = nullptr;
  int bank_count = 0;        // matrices in the bank: an expert id outside [0, bank_count) is clamped (checked build: reported)
  const int32_t* expert_ids_dev = nullptr;
  int x_row_div = 1;             // activation row of pair p = p / x_row_div
  const float* row_scale_dev = nullptr;  // optional per-pair output scale (router gate)
  // EPI_QKV_ROPE: rows are [allQ | allK | allV]; Q pairs are rotated and stored to y, K pairs are rotated and
  // stored straight into the cache at slot cache_len[b], V rows go to the cache unrotated (RoPE + KV append fused)
  const float* rope_cs = nullptr;        // [B][head_dim/2][2] cos, sin of this step
  int rope_q_width = 0, rope_kv_width = 0, rope_head_dim = 0, rope_kv_heads = 0, rope_max_ctx = 0;
  float* k_cache = nullptr;
  float* v_cache = nullptr;
  int k_blocked = 0;                     // K cache in the block-transposed layout (cai_k_blocked_index)
  const int32_t* cache_len_dev = nullptr;
  const float* norm_gain = nullptr;      // fuse y = W (gain * x * inv_rms(x)): the preceding TNNetTokenRMSNorm
  float norm_eps = 0.f;
};
// true when linear_launch can apply the RMSNorm itself for this weight and batch
bool linear_can_fuse_norm(const QWeight* w, int batch);

int linear_launch(cai_ctx* ctx, const LinearArgs& a);
int cai_check_device_error(cai_ctx* ctx);   // CAI_ERR_CUDA if a kernel raised the error word

// ops.cu
int op_embed(cai_ctx* ctx, const QWeight* table, const int32_t* tokens_dev, int batch, float* out, int64_t ld);
int op_rmsnorm(cai_ctx* ctx, const float* x, int64_t ldx, const float* gain, float* y, int64_t ldy, int tokens, int depth, float eps);
int op_rope(cai_ctx* ctx, float* x, int64_t ldx, int tokens, int depth, int head_dim, const float* theta_dev,
            const int32_t* pos_dev, int pos_stride, int pos_offset);
int op_swiglu(cai_ctx* ctx, const float* x, int64_t ldx, float* y, int64_t ldy, int tokens, int half);
int op_topk_gate(cai_ctx* ctx, const float* logits, int tokens, int n_experts, int top_k, int renorm,
                 int32_t* ids, float* gates);
#define CAI_ARGMAX_CHUNKS 128
int op_argmax(cai_ctx* ctx, const float* logits, int64_t ld, int batch, int n, int32_t* out_idx, float* out_val,
              float* part_val, int* part_idx, int* tickets);   // scratch: [batch][CAI_ARGMAX_CHUNKS] x2, tickets [batch] zeroed once
int op_rope_table(cai_ctx* ctx, const float* theta_dev, const int32_t* pos_dev, int batch, int half, float* cs_dev);
// pairs whose expert lies outside [expert_lo, expert_hi) are left out (expert parallelism: another rank owns them)
int op_moe_group(cai_ctx* ctx, const int32_t* expert_ids, int pairs, int n_experts, int tile_rows, int max_tiles,
                 int32_t* tile_expert, int32_t* tile_pairs, int expert_lo, int expert_hi);
// expert parallelism: packs a rank's rows [hidden floats | top_k expert ids | top_k gates] for one all-gather, and the
// partial combine  y[t][:] = sum over the slots of token t whose expert is in [lo, hi) of gate * pair_out[pair][:]
int op_moe_pack(cai_ctx* ctx, const float* h, int64_t ldh, const int32_t* ids, const float* gates, int tokens, int hidden, int top_k, int stride,
                float* packed);
int op_moe_unpack_ids(cai_ctx* ctx, const float* packed, int tokens, int hidden, int top_k, int stride, int32_t* ids, float* gates);
int op_moe_combine_partial(cai_ctx* ctx, const float* pair_out, int64_t ldp, const int32_t* ids, const float* gates, int tokens, int top_k,
                           int hidden, int expert_lo, int expert_hi, float* y, int64_t ldy);
int op_add_rows(cai_ctx* ctx, float* x, int64_t ldx, const float* y, int64_t ldy, int tokens, int width);
// gemm_tc.cu: grouped tensor-core GEMM over the tiles op_moe_group made (16 pairs per tile)
size_t gemm_tc_group_tile_bytes(int64_t k);
int gemm_tc_launch_grouped(cai_ctx* ctx, int type, const void* const* bank_codes, const __half* const* bank_scales, int64_t n, int64_t k,
                           int64_t sstride, const float* x, int64_t ldx, int x_row_div, float* y, int64_t ldy,
                           const int32_t* tile_expert, const int32_t* tile_pairs, int n_tiles, void* xp_tiles, float* unscale_tiles);
int op_moe_combine(cai_ctx* ctx, float* x, int64_t ldx, const float* pair_out, int64_t ldp, const float* gates,
                   int tokens, int top_k, int depth);
int op_add_inplace(cai_ctx* ctx, float* x, const float* y, int64_t n);
int op_rope_theta_table(cai_ctx* ctx, float* theta_dev, int head_dim, float base);

// attention.cu
struct AttnArgs {
  float* qkv = nullptr;         // [B][ld]: [allQ | allK | allV] rows; Q and K are normed/rotated in place
  int64_t ld = 0;
  float* k_cache = nullptr;     // [B][kv_heads][max_ctx][hd], head-major per sequence
  float* v_cache = nullptr;
  const int32_t* cache_len_dev = nullptr;  // [B] length BEFORE this step (slot to append at)
  int batch = 1, q_heads = 0, kv_heads = 0, head_dim = 0, max_ctx = 0;
  const float* theta = nullptr;            // [hd/2] RoPE frequencies; NULL = rows are already rotated
  const int32_t* pos_dev = nullptr;        // [B] absolute positions (NULL = cache length)
  const float* q_norm = nullptr;           // optional full-width RMSNorm gains applied before RoPE
  const float* k_norm = nullptr;
  float eps = 0.f;
  float* out = nullptr;         // [B][ldo]
  int64_t ldo = 0;
  float* partial = nullptr;     // scratch: [B][q_heads][nsplit][hd + 2]
  int nsplit = 1;
  // int8 KV cache (set k_codes to use it; k_cache / v_cache are then ignored): codes [B][kv_heads][max_ctx][hd],
  // one fp32 scale per (sequence, kv head, position) row [B][kv_heads][max_ctx]
  int8_t* k_codes = nullptr;
  int8_t* v_codes = nullptr;
  float* k_scales = nullptr;
  float* v_scales = nullptr;
  // K cache layout: 0 = [pos][d] rows as the reference keeps them (neural/neural.cl:2343-2346), 1 = block-transposed
  // (cai_k_blocked_index; sessions use it, max_ctx must then be a multiple of 32 and head_dim of 4)
  int k_blocked = 0;
  // rows a step sees: sliding window (> 0: the most recent `window` rows) or StreamingLLM eviction (evict_window > 0: the
  // first evict_sinks rows + the most recent evict_window rows, kept as sinks + a ring)
  int window = 0, evict_sinks = 0, evict_window = 0;
  // optional: row r of the batch belongs to sequence seq_index[r] of the cache (several rows may be consecutive
  // positions of ONE sequence: chunked prefill); NULL = row r is sequence r. cache_len_dev stays per row.
  const int32_t* seq_index_dev = nullptr;
};
int attn_nsplit(cai_ctx* ctx, int batch, int kv_heads, int max_ctx);
size_t attn_partial_floats(int batch, int q_heads, int nsplit, int head_dim);
bool attn_int8_supported(int q_heads, int kv_heads, int head_dim);
bool attn_k_blocked_supported(int q_heads, int kv_heads, int head_dim);
int attn_rope_append(cai_ctx* ctx, const AttnArgs& a);
int attn_decode(cai_ctx* ctx, const AttnArgs& a);

// sample.cu
int sample_scratch_floats(int batch);
int sample_launch(cai_ctx* ctx, const float* logits, int64_t ld, int batch, int vocab, int k, float temperature, float top_p,
                  unsigned long long seed, const float* uniforms_dev, float* scratch, int32_t* ids_out_dev, float* probs_out_dev,
                  int32_t* tokens_dev, int32_t* trace_dev, const int32_t* trace_count_dev, long long trace_cap, int32_t* drawn_out_dev);

// comm.cu
int comm_allreduce(cai_ctx* ctx, float* buf, int64_t count);
int comm_allgather(cai_ctx* ctx, const float* send, float* recv, int64_t count_per_rank);
int comm_reduce_scatter(cai_ctx* ctx, const float* send, float* recv, int64_t count_per_rank);
int comm_world(cai_ctx* ctx);
int comm_rank(cai_ctx* ctx);
struct cai_tp_ar;   // one-shot all-reduce over peer memory (comm.cu)
int comm_ar_create(cai_ctx* ctx, int sites, int64_t max_elems, cai_tp_ar** out);   // collective; *out stays NULL when peers cannot be mapped
void comm_ar_destroy(cai_ctx* ctx, cai_tp_ar* ar);                                 // collective
float* comm_ar_slot(cai_tp_ar* ar, int site);
int comm_ar_reduce(cai_ctx* ctx, cai_tp_ar* ar, int site, int64_t n, const float* resid, float* out);
// expert-parallel dispatch / combine over the same slots (comm.cu)
int comm_ep_dispatch(cai_ctx* ctx, cai_tp_ar* ar, int site, int tokens, int stride, int hidden, int top_k, int expert_lo, int expert_hi,
                     float* all, int32_t* ids_out, float* gates_out);
int comm_ep_combine(cai_ctx* ctx, cai_tp_ar* ar, int site, int tokens, int hidden, int top_k, int experts_per_rank, const int32_t* my_ids,
                    float* x, int64_t ldx);
void comm_destroy(cai_ctx* ctx);

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
// Block-transposed K cache of a session (one KV head): positions in blocks of 32; inside a block the 16-byte piece
// (4 channels) p of position r lies at float offset (p * 32 + r) * 4. The decode kernels walk K with "lane = position":
// in this layout the 32 lanes of a warp read 512 contiguous bytes per instruction, and a block's pieces 8 s .. 8 s + 7
// are one contiguous 4 KB run that an asynchronous copy can land in shared memory as it is. (The reference's row
// layout [pos][d] makes the same access 32 separate 512-byte-strided pieces.) V keeps the row layout: it is walked
// with "lane = channels".
// The int8 cache's K codes, same idea with 16-byte pieces of 16 codes: byte offset of code d of position pos.
__host__ __device__ __forceinline__ size_t cai_k_blocked_index_i8(int pos, int d, int head_dim) {
  return ((size_t)(pos >> 5) * (size_t)(head_dim >> 4) + (size_t)(d >> 4)) * 512 + (size_t)(pos & 31) * 16 + (size_t)(d & 15);
}
__host__ __device__ __forceinline__ size_t cai_k_blocked_index(int pos, int d, int head_dim) {
  return ((size_t)(pos >> 5) * (size_t)(head_dim >> 2) + (size_t)(d >> 2)) * 128 + (size_t)(pos & 31) * 4 + (size_t)(d & 3);
}
// Programmatic dependent launch. A kernel launched through pdl_launch may start while the kernel
// before it in the stream is still running; it must call pdl_wait() before it touches anything that
// kernel wrote (pdl_wait returns once the previous kernel has completed and its writes are visible),
// and may do independent work (barrier set-up, weight prefetch) before that. pdl_trigger() lets the
// NEXT kernel start early in the same way. Both are no-ops for ordinarily launched kernels.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t pdl_launch(cai_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ctx->use_pdl ? 1 : 0;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// Nanoseconds of the GPU's global timer: the clock the bounded waits measure themselves against.
__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; every thread gets the result. `red` needs 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
// Block-wide maximum of non-negative values; every thread gets the result.
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_max(t);
  return t;
}
// int8 code in byte `i` of a word whose bytes were XOR-ed with 0x80 -> float, exactly.
// (0x4B000000 | u) is the float 8388608 + u; subtracting 8388736 leaves u - 128.
__device__ __forceinline__ float biased_byte_to_float(uint32_t w, int i) {
  uint32_t bits = __byte_perm(w, 0x4B000000u, 0x7650u + (uint32_t)i);
  return __uint_as_float(bits) - 8388736.0f;
}
// unsigned byte `i` of w minus `bias` -> float, exactly.
__device__ __forceinline__ float ubyte_to_float(uint32_t w, int i, float magic_plus_bias) {
  uint32_t bits = __byte_perm(w, 0x4B000000u, 0x7650u + (uint32_t)i);
  return __uint_as_float(bits) - magic_plus_bias;
}
#endif
