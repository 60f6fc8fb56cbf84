// Multi-GPU plumbing: one process per GPU, NCCL communicator on the context's stream.
#include "cai_common.cuh"
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

extern "C" {

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
