// Multi-GPU plumbing: one process per GPU, NCCL communicator on the context's stream.
#include "cai_common.cuh"
#include "step_kernel.cuh"
#include <nccl.h>

struct cai_comm_state {
  ncclComm_t comm;
  int rank, world;
};

#define CAI_NCCL(ctx, call)                                                                          \
  do {                                                                                               \
    ncclResult_t r__ = (call);                                                                       \
    if (r__ != ncclSuccess)                                                                          \
      return cai_fail((ctx), CAI_ERR_COMM, "%s -> %s (%s:%d)", #call, ncclGetErrorString(r__), __FILE__, __LINE__); \
  } while (0)

int comm_world(cai_ctx* ctx) { return ctx->comm ? ctx->comm->world : 1; }
int comm_rank(cai_ctx* ctx) { return ctx->comm ? ctx->comm->rank : 0; }

void comm_destroy(cai_ctx* ctx) {
  if (ctx->comm) {
    ncclCommDestroy(ctx->comm->comm);
    delete ctx->comm;
    ctx->comm = nullptr;
  }
}

int comm_allreduce(cai_ctx* ctx, float* buf, int64_t count) {
  if (!ctx->comm) return cai_fail(ctx, CAI_ERR_STATE, "communicator not initialised");
  CAI_NCCL(ctx, ncclAllReduce(buf, buf, (size_t)count, ncclFloat, ncclSum, ctx->comm->comm, ctx->stream));
  if (ctx->prof_on) cai_prof_mark(ctx, FAM_COMM);
  return CAI_OK;
}

int comm_allgather(cai_ctx* ctx, const float* send, float* recv, int64_t count_per_rank) {
  if (!ctx->comm) return cai_fail(ctx, CAI_ERR_STATE, "communicator not initialised");
  CAI_NCCL(ctx, ncclAllGather(send, recv, (size_t)count_per_rank, ncclFloat, ctx->comm->comm, ctx->stream));
  if (ctx->prof_on) cai_prof_mark(ctx, FAM_COMM);
  return CAI_OK;
}

// recv[rank's slice of count_per_rank floats] = sum over ranks of send[that slice]
int comm_reduce_scatter(cai_ctx* ctx, const float* send, float* recv, int64_t count_per_rank) {
  if (!ctx->comm) return cai_fail(ctx, CAI_ERR_STATE, "communicator not initialised");
  CAI_NCCL(ctx, ncclReduceScatter(send, recv, (size_t)count_per_rank, ncclFloat, ncclSum, ctx->comm->comm, ctx->stream));
  if (ctx->prof_on) cai_prof_mark(ctx, FAM_COMM);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// One-shot all-reduce over NVLink peer memory, fused with the residual add.
//
// Tensor-parallel decode sums a [batch, hidden] partial result over the ranks twice per layer; at
// batch 1 that is 20 KB per rank, where a library all-reduce costs its fixed latency. Here every rank
// keeps its partial results in a buffer the other ranks map (CUDA IPC); the row-parallel GEMV writes
// its partial straight into that buffer, then ONE small kernel per rank
//   1. stores this call's sequence number into every rank's flag word (a remote store),
//   2. waits (bounded) until all ranks' flags show the number,
//   3. loads every rank's partial with plain peer loads and adds them in rank order to the residual.
// All ranks add in the same order, so they stay bit-identical. Every call site of a step owns its slot
// of the buffer: a slot is rewritten one step later, after at least one more all-reduce, which a rank
// only passes once every peer has finished reading the earlier slots. No cluster-scope copies, no
// switch reduction: plain ld/st over mapped peer memory.
// ---------------------------------------------------------------------------
struct cai_tp_ar {
  char* block = nullptr;          // [flags: 64 ints][slots: sites * max_elems floats], cudaMalloc'd, IPC-exported
  void* peer_block[8] = {nullptr};
  int* seq_dev = nullptr;         // [0] calls completed so far, [1] "a wait ran out" word
  int* ticket_dev = nullptr;
  int sites = 0;
  int64_t max_elems = 0;
  int rank = 0, world = 1;
};
static const size_t AR_FLAG_BYTES = 256;

struct ArParams {
  const float* peer_slot[8];
  int* peer_flags[8];
  int* my_flags;
  int* seq;
  int* ticket;
  int rank, world, n4;
  const float4* resid;
  float4* out;
  int* err;
  int* gave_up;            // device word of this rank: set by the first wait that ran out
  unsigned wait_limit_us;
};

__global__ void tp_allreduce_kernel(const ArParams p) {
  __shared__ int s_seq;
  if (threadIdx.x == 0) s_seq = *(volatile int*)p.seq + 1;
  __syncthreads();
  const int seq = s_seq;
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();                                   // this rank's partial (written by the previous kernel) first
    *(volatile int*)(p.peer_flags[threadIdx.x] + p.rank) = seq;
  }
  if (threadIdx.x < p.world) {
    // Bounded wait, measured on the global timer. Once a wait of this rank has run out, later calls do not wait
    // again (a missing peer must cost one time limit, not one per call site of every step).
    const volatile int* f = (const volatile int*)(p.my_flags + threadIdx.x);
    bool ok = *f >= seq;
    if (!ok && *(volatile int*)p.gave_up == 0) {
      const unsigned long long t0 = gtime_ns(), limit = (unsigned long long)p.wait_limit_us * 1000ull;
      while (true) {
        if (*f >= seq) { ok = true; break; }
        if (gtime_ns() - t0 > limit) break;
      }
    }
    if (!ok) { *p.err = 1; *(volatile int*)p.gave_up = 1; }   // give up: the host sees the error word
  }
  __syncthreads();
  __threadfence_system();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.n4; i += gridDim.x * blockDim.x) {
    float4 acc = p.resid ? p.resid[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < p.world; ++r) {
      float4 v;
      const float4* src = (const float4*)p.peer_slot[r] + i;
      asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    p.out[i] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(p.ticket, 1);
    if (old == (int)gridDim.x - 1) { *p.ticket = 0; *(volatile int*)p.seq = seq; }
  }
}

// ---------------------------------------------------------------------------
// Expert-parallel exchange over the same peer-mapped slots: the dispatch and the combine of a mixture-of-experts
// layer as two kernels instead of two library collectives.
//   dispatch  every rank has packed its tokens' rows [hidden | top_k ids | top_k gates] into its own slot. After the
//             arrival exchange (same sequence-numbered flags as above) a rank pulls, from every peer, the ids and
//             gates of all tokens and the hidden row of those tokens that route to at least one of ITS experts - the
//             others never reach a tile, so their rows stay unread (at 8 ranks and top-8 of 64 experts a third of them).
//   combine   every rank has written, for all tokens, the gate-weighted sum over its own experts into its slot. The
//             owner of a token adds, in rank order, the sums of the ranks that host one of the token's experts to the
//             residual stream (bit-identical whatever the rank count's timing; no atomics).
// A slot is rewritten one step later, after 2 x layers - 1 further exchanges, which a rank only passes once every peer
// has finished the earlier ones. Plain ld / st over mapped peer memory; every wait is bounded on the global timer.
// ---------------------------------------------------------------------------
struct EpParams {
  const float* peer_slot[8];
  int* peer_flags[8];
  int* my_flags;
  int* seq;
  int* ticket;
  int* err;
  int* gave_up;
  unsigned wait_limit_us;
  int rank, world;
  int tokens, stride, hidden, top_k;     // tokens per rank; floats per packed row
  int expert_lo, expert_hi, experts_per_rank;
  float* all;                            // dispatch: [world * tokens][stride] gathered rows
  int32_t* ids_out; float* gates_out;    // dispatch: [world * tokens][top_k]
  float* x; int64_t ldx;                 // combine: residual stream of this rank's tokens, updated in place
  const int32_t* my_ids;                 // combine: [tokens][top_k] expert ids of this rank's tokens
};

// arrival exchange of one call: returns the call's sequence number (every thread), false in *ok when a wait ran out
__device__ __forceinline__ int ep_arrive_and_wait(const EpParams& p, int* s_seq) {
  if (threadIdx.x == 0) *s_seq = *(volatile int*)p.seq + 1;
  __syncthreads();
  const int seq = *s_seq;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < p.world) {
    __threadfence_system();                                   // this rank's slot (written by the previous kernel) first
    *(volatile int*)(p.peer_flags[threadIdx.x] + p.rank) = seq;
  }
  if (threadIdx.x < p.world) {
    const volatile int* f = (const volatile int*)(p.my_flags + threadIdx.x);
    bool ok = *f >= seq;
    if (!ok && *(volatile int*)p.gave_up == 0) {
      const unsigned long long t0 = gtime_ns(), limit = (unsigned long long)p.wait_limit_us * 1000ull;
      while (true) {
        if (*f >= seq) { ok = true; break; }
        if (gtime_ns() - t0 > limit) break;
      }
    }
    if (!ok) { *p.err = 1; *(volatile int*)p.gave_up = 1; }
  }
  __syncthreads();
  __threadfence_system();
  return seq;
}
__device__ __forceinline__ void ep_finish(const EpParams& p, int seq) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(p.ticket, 1);
    if (old == (int)(gridDim.x * gridDim.y) - 1) { *p.ticket = 0; *(volatile int*)p.seq = seq; }
  }
}
__device__ __forceinline__ float4 ep_ld4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// grid.x = world * tokens (one CTA per gathered row)
__global__ void ep_dispatch_kernel(const EpParams p) {
  __shared__ int s_seq;
  __shared__ int s_need;
  const int seq = ep_arrive_and_wait(p, &s_seq);
  const int row = blockIdx.x;
  const int r = row / p.tokens, t = row - r * p.tokens;
  const float* src = p.peer_slot[r] + (size_t)t * p.stride;
  float* dst = p.all + (size_t)row * p.stride;
  if (threadIdx.x == 0) s_need = 0;
  __syncthreads();
  if (threadIdx.x < p.top_k) {
    float idf, g;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(idf) : "l"(src + p.hidden + threadIdx.x));
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(g) : "l"(src + p.hidden + p.top_k + threadIdx.x));
    const int e = __float_as_int(idf);
    dst[p.hidden + threadIdx.x] = idf;
    dst[p.hidden + p.top_k + threadIdx.x] = g;
    p.ids_out[row * p.top_k + threadIdx.x] = e;
    p.gates_out[row * p.top_k + threadIdx.x] = g;
    if (e >= p.expert_lo && e < p.expert_hi) s_need = 1;
  }
  __syncthreads();
  if (s_need) {
    // a remote load costs ~2 us: a thread requests its pieces (up to four) together, then stores them
    for (int c0 = threadIdx.x * 4; c0 < p.hidden; c0 += blockDim.x * 16) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x * 4;
        if (c < p.hidden) v[u] = ep_ld4(src + c);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x * 4;
        if (c < p.hidden) *(float4*)(dst + c) = v[u];
      }
    }
  }
  ep_finish(p, seq);
}

// grid = (tokens, column blocks): x[t] += sum in rank order of the partial sums of the ranks that host one of t's experts
__global__ void ep_combine_kernel(const EpParams p) {
  __shared__ int s_seq;
  __shared__ int s_mask;
  const int seq = ep_arrive_and_wait(p, &s_seq);
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int mask = 0;
    for (int k = 0; k < p.top_k; ++k) {
      const int e = p.my_ids[t * p.top_k + k];
      if (e >= 0) mask |= 1 << (e / p.experts_per_rank);
    }
    s_mask = mask;
  }
  __syncthreads();
  const int mask = s_mask;
  const size_t grow = (size_t)(p.rank * p.tokens + t) * (size_t)p.hidden;
  const int cols_per_block = (((p.hidden / 4) + gridDim.y - 1) / gridDim.y) * 4;
  const int c_begin = blockIdx.y * cols_per_block;
  int c_end = c_begin + cols_per_block; if (c_end > p.hidden) c_end = p.hidden;
  for (int c = c_begin + threadIdx.x * 4; c < c_end; c += blockDim.x * 4) {
    // all ranks' pieces are requested together (a remote load costs ~2 us), then added in rank order
    float4 v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.world && ((mask >> r) & 1)) v[r] = ep_ld4(p.peer_slot[r] + grow + c);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.world && ((mask >> r) & 1)) { sum.x += v[r].x; sum.y += v[r].y; sum.z += v[r].z; sum.w += v[r].w; }
    float4* xp = (float4*)(p.x + (int64_t)t * p.ldx + c);
    float4 xv = *xp;
    xv.x += sum.x; xv.y += sum.y; xv.z += sum.z; xv.w += sum.w;
    *xp = xv;
  }
  ep_finish(p, seq);
}

static void ep_fill(EpParams& p, cai_ctx* ctx, cai_tp_ar* ar, int site) {
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < ar->world; ++r) {
    p.peer_flags[r] = (int*)ar->peer_block[r];
    p.peer_slot[r] = (const float*)((char*)ar->peer_block[r] + AR_FLAG_BYTES) + (size_t)site * (size_t)ar->max_elems;
  }
  p.my_flags = (int*)ar->block; p.seq = ar->seq_dev; p.gave_up = ar->seq_dev + 1; p.ticket = ar->ticket_dev;
  p.rank = ar->rank; p.world = ar->world; p.err = ctx->err_flag; p.wait_limit_us = ctx->wait_limit_us;
}

int comm_ep_dispatch(cai_ctx* ctx, cai_tp_ar* ar, int site, int tokens, int stride, int hidden, int top_k, int expert_lo, int expert_hi,
                     float* all, int32_t* ids_out, float* gates_out) {
  if (site < 0 || site >= ar->sites || (int64_t)tokens * stride > ar->max_elems || (hidden % 4) || (stride % 4) || top_k > 256)
    return cai_fail(ctx, CAI_ERR_INVALID, "expert dispatch: slot %d of %d, %d rows of %d", site, ar->sites, tokens, stride);
  EpParams p;
  ep_fill(p, ctx, ar, site);
  p.tokens = tokens; p.stride = stride; p.hidden = hidden; p.top_k = top_k; p.expert_lo = expert_lo; p.expert_hi = expert_hi;
  p.all = all; p.ids_out = ids_out; p.gates_out = gates_out;
  ctx->cur_family = FAM_COMM;
  ep_dispatch_kernel<<<dim3((unsigned)(ar->world * tokens)), 256, 0, ctx->stream>>>(p);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

int comm_ep_combine(cai_ctx* ctx, cai_tp_ar* ar, int site, int tokens, int hidden, int top_k, int experts_per_rank, const int32_t* my_ids,
                    float* x, int64_t ldx) {
  if (site < 0 || site >= ar->sites || (int64_t)ar->world * tokens * hidden > ar->max_elems || (hidden % 4) || (ldx % 4))
    return cai_fail(ctx, CAI_ERR_INVALID, "expert combine: slot %d of %d, %d rows of %d", site, ar->sites, ar->world * tokens, hidden);
  EpParams p;
  ep_fill(p, ctx, ar, site);
  p.tokens = tokens; p.hidden = hidden; p.top_k = top_k; p.experts_per_rank = experts_per_rank; p.my_ids = my_ids; p.x = x; p.ldx = ldx;
  int yblocks = (2 * ctx->sm_count) / (tokens > 0 ? tokens : 1);
  if (yblocks < 1) yblocks = 1;
  if (yblocks > 8) yblocks = 8;
  ctx->cur_family = FAM_COMM;
  ep_combine_kernel<<<dim3((unsigned)tokens, (unsigned)yblocks), 256, 0, ctx->stream>>>(p);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

void comm_ar_destroy(cai_ctx* ctx, cai_tp_ar* ar) {
  if (!ar) return;
  // every rank must have finished reading before any rank unmaps or frees
  if (ctx->comm && ar->seq_dev) {
    ncclAllReduce(ar->seq_dev, ar->seq_dev, 1, ncclInt, ncclMax, ctx->comm->comm, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
  }
  for (int r = 0; r < ar->world; ++r)
    if (r != ar->rank && ar->peer_block[r]) cudaIpcCloseMemHandle(ar->peer_block[r]);
  if (ar->block) cudaFree(ar->block);
  if (ar->seq_dev) cudaFree(ar->seq_dev);
  if (ar->ticket_dev) cudaFree(ar->ticket_dev);
  delete ar;
}

// Collective over the communicator: every rank calls it with the same arguments.
int comm_ar_create(cai_ctx* ctx, int sites, int64_t max_elems, cai_tp_ar** out) {
  *out = nullptr;
  if (!ctx->comm) return cai_fail(ctx, CAI_ERR_STATE, "communicator not initialised");
  const char* mode = getenv("CAI_TP_ALLREDUCE");
  if (mode && !strcmp(mode, "nccl")) return CAI_OK;           // caller falls back to the library collectives
  const int world = ctx->comm->world, rank = ctx->comm->rank;
  if (world > 8 || (max_elems % 4)) return CAI_OK;
  cai_tp_ar* ar = new cai_tp_ar();
  ar->sites = sites; ar->max_elems = max_elems; ar->rank = rank; ar->world = world;
  const size_t bytes = AR_FLAG_BYTES + (size_t)sites * (size_t)max_elems * sizeof(float);
  cudaIpcMemHandle_t mine;
  memset(&mine, 0, sizeof(mine));
  cudaIpcMemHandle_t* all_dev = nullptr;
  std::vector<cudaIpcMemHandle_t> all((size_t)world);
  int ok = 1;
  if (cudaMalloc((void**)&ar->block, bytes) != cudaSuccess || cudaMemset(ar->block, 0, bytes) != cudaSuccess ||
      cudaMalloc((void**)&ar->seq_dev, 8) != cudaSuccess || cudaMemset(ar->seq_dev, 0, 8) != cudaSuccess ||
      cudaMalloc((void**)&ar->ticket_dev, 4) != cudaSuccess || cudaMemset(ar->ticket_dev, 0, 4) != cudaSuccess ||
      cudaIpcGetMemHandle(&mine, ar->block) != cudaSuccess)
    ok = 0;
  cudaGetLastError();
  // The handle exchange is collective and must run on every rank whatever happened above, or the others would be left
  // waiting inside the library: it goes through the context's upload staging buffer (allocated at start-up or here;
  // if even that fails the rank has no device memory at all and the communicator is lost anyway).
  if (cai_ensure_staging(ctx, sizeof(cudaIpcMemHandle_t) * (size_t)world) == CAI_OK) all_dev = (cudaIpcMemHandle_t*)ctx->staging_dev;
  else ok = 0;
  if (all_dev) {
    cudaMemcpy(all_dev + rank, &mine, sizeof(mine), cudaMemcpyHostToDevice);
    if (ncclAllGather(all_dev + rank, all_dev, sizeof(cudaIpcMemHandle_t), ncclInt8, ctx->comm->comm, ctx->stream) != ncclSuccess) ok = 0;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) ok = 0;
    if (ok) cudaMemcpy(all.data(), all_dev, sizeof(cudaIpcMemHandle_t) * (size_t)world, cudaMemcpyDeviceToHost);
  }
  if (ok) {
    ar->peer_block[rank] = ar->block;
    for (int r = 0; r < world && ok; ++r) {
      if (r == rank) continue;
      if (cudaIpcOpenMemHandle(&ar->peer_block[r], all[(size_t)r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { ar->peer_block[r] = nullptr; ok = 0; }
    }
    cudaGetLastError();
  }
  // agree on the outcome: one rank without peer mappings sends everybody to the library path
  int* agree = nullptr;
  int all_ok = 0;
  if (cudaMalloc((void**)&agree, 4) == cudaSuccess) {
    cudaMemcpy(agree, &ok, 4, cudaMemcpyHostToDevice);
    ncclAllReduce(agree, agree, 1, ncclInt, ncclMin, ctx->comm->comm, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(&all_ok, agree, 4, cudaMemcpyDeviceToHost);
    cudaFree(agree);
  }
  if (!all_ok) { comm_ar_destroy(ctx, ar); return CAI_OK; }
  *out = ar;
  return CAI_OK;
}

// The raw view of the exchange buffers for kernels that do the flag protocol themselves (the persistent step kernel).
int comm_ar_exchange(cai_tp_ar* ar, TpExchange* out) {
  if (!ar || !out) return CAI_ERR_INVALID;
  memset(out, 0, sizeof(*out));
  out->rank = ar->rank; out->world = ar->world;
  out->my_flags = (int*)ar->block;
  out->my_slots = (float*)(ar->block + AR_FLAG_BYTES);
  for (int r = 0; r < ar->world; ++r) {
    out->peer_flags[r] = (int*)ar->peer_block[r];
    out->peer_slots[r] = (const float*)((char*)ar->peer_block[r] + AR_FLAG_BYTES);
  }
  out->max_elems = ar->max_elems; out->sites = ar->sites;
  out->seq = ar->seq_dev; out->gave_up = ar->seq_dev + 1;
  return CAI_OK;
}

float* comm_ar_slot(cai_tp_ar* ar, int site) {
  return (float*)(ar->block + AR_FLAG_BYTES) + (size_t)site * (size_t)ar->max_elems;
}

// out = resid + sum over ranks of slot[site] (resid may be NULL); n floats, n % 4 == 0.
int comm_ar_reduce(cai_ctx* ctx, cai_tp_ar* ar, int site, int64_t n, const float* resid, float* out) {
  if (site < 0 || site >= ar->sites || n > ar->max_elems || (n % 4)) return cai_fail(ctx, CAI_ERR_INVALID, "all-reduce slot %d of %d, %lld elements", site, ar->sites, (long long)n);
  ArParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < ar->world; ++r) {
    p.peer_flags[r] = (int*)ar->peer_block[r];
    p.peer_slot[r] = (const float*)((char*)ar->peer_block[r] + AR_FLAG_BYTES) + (size_t)site * (size_t)ar->max_elems;
  }
  p.my_flags = (int*)ar->block; p.seq = ar->seq_dev; p.gave_up = ar->seq_dev + 1; p.ticket = ar->ticket_dev;
  p.rank = ar->rank; p.world = ar->world; p.n4 = (int)(n / 4);
  p.resid = (const float4*)resid; p.out = (float4*)out; p.err = ctx->err_flag; p.wait_limit_us = ctx->wait_limit_us;
  // one 16-byte element per thread while that fits the machine: a remote load costs ~2 us, so a thread should not
  // walk many of them (at batch 64 the 16-block cap this used to have made a 1.3 MB reduction take ~60 us)
  int blocks = (p.n4 + 255) / 256;
  if (blocks > 2 * ctx->sm_count) blocks = 2 * ctx->sm_count;
  if (blocks < 1) blocks = 1;
  ctx->cur_family = FAM_COMM;
  tp_allreduce_kernel<<<blocks, 256, 0, ctx->stream>>>(p);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

int step_barrier_selftest(cai_ctx* ctx, unsigned limit_us);   // step_kernel.cu

extern "C" {

// Makes a device-side bounded wait run out on purpose, without any peer and without hanging anything:
//   which = 0: the tensor-parallel all-reduce kernel as rank 0 of a world of 2 whose second rank does not exist (its
//              arrival word is a local buffer nobody writes);
//   which = 1: the grid barrier of the persistent step kernel with one arrival more expected than CTAs launched.
// Each gives up after limit_us, raises the context's error word and returns; the status is what the next
// synchronizing call would report (CAI_ERR_CUDA when the time-out path worked).
int cai_selftest_wait_timeout(cai_ctx* ctx, int which, unsigned limit_us) {
  CAI_TRY(cai_bind(ctx));
  if (limit_us < 1 || limit_us > 5000000) return cai_fail(ctx, CAI_ERR_INVALID, "cai_selftest_wait_timeout: limit %u us outside 1..5000000", limit_us);
  if (which == 1) return step_barrier_selftest(ctx, limit_us);
  if (which != 0) return cai_fail(ctx, CAI_ERR_INVALID, "cai_selftest_wait_timeout: which = %d", which);
  char* buf = nullptr;
  const size_t bytes = 2 * AR_FLAG_BYTES + 2 * 64 * sizeof(float) + 64;
  CAI_CUDA(ctx, cudaMalloc((void**)&buf, bytes));
  CAI_CUDA(ctx, cudaMemsetAsync(buf, 0, bytes, ctx->stream));
  ArParams p;
  memset(&p, 0, sizeof(p));
  p.my_flags = (int*)buf;                              // [0] is raised by the kernel itself, [1] by nobody
  p.peer_flags[0] = (int*)buf;
  p.peer_flags[1] = (int*)(buf + AR_FLAG_BYTES);       // the missing rank's words: local, never read
  p.peer_slot[0] = (const float*)(buf + 2 * AR_FLAG_BYTES);
  p.peer_slot[1] = p.peer_slot[0] + 64;
  p.seq = (int*)(buf + 2 * AR_FLAG_BYTES + 2 * 64 * sizeof(float));
  p.gave_up = p.seq + 1; p.ticket = p.seq + 2;
  p.rank = 0; p.world = 2; p.n4 = 16;
  p.resid = nullptr; p.out = (float4*)(buf + 2 * AR_FLAG_BYTES);
  p.err = ctx->err_flag; p.wait_limit_us = limit_us;
  tp_allreduce_kernel<<<1, 256, 0, ctx->stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFree(buf);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "all-reduce self-test -> %s", cudaGetErrorString(e));
  ctx->launches++;
  return cai_check_device_error(ctx);
}

int cai_comm_unique_id(unsigned char out_id[128]) {
  if (!out_id) return CAI_ERR_INVALID;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return CAI_ERR_COMM;
  memcpy(out_id, &id, 128);
  return CAI_OK;
}

int cai_comm_init(cai_ctx* ctx, int rank, int world, const unsigned char id[128]) {
  CAI_TRY(cai_bind(ctx));
  if (!id || world < 1 || rank < 0 || rank >= world) return cai_fail(ctx, CAI_ERR_INVALID, "cai_comm_init: rank %d of %d", rank, world);
  if (ctx->comm) return cai_fail(ctx, CAI_ERR_STATE, "communicator already initialised");
  ncclUniqueId uid;
  memcpy(&uid, id, 128);
  cai_comm_state* c = new cai_comm_state();
  c->rank = rank; c->world = world;
  ncclResult_t r = ncclCommInitRank(&c->comm, world, uid, rank);
  if (r != ncclSuccess) { delete c; return cai_fail(ctx, CAI_ERR_COMM, "ncclCommInitRank -> %s", ncclGetErrorString(r)); }
  ctx->comm = c;
  return CAI_OK;
}

int cai_comm_allreduce_dev(cai_ctx* ctx, float* buf_dev, int64_t count) {
  CAI_TRY(cai_bind(ctx));
  if (!buf_dev || count < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_comm_allreduce_dev: bad argument");
  CAI_TRY(comm_allreduce(ctx, buf_dev, count));
  return CAI_OK;
}

}  // extern "C"
