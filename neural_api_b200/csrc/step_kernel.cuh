// One persistent kernel per decode step (dense models, one sequence, Q8_0 weights, fp32 KV cache).
// model.cu fills a StepSetup from a session; step_kernel.cu turns it into a plan and launches it.
#pragma once
#include "cai_common.cuh"

struct StepLayerSetup {
  const QWeight *wqkv, *wo, *wgu, *wdown;
  const float *attn_norm, *ffn_norm;
  float *k_cache, *v_cache;           // this layer's [kv_heads][max_ctx][head_dim]
};

struct cai_tp_ar;

struct StepSetup {
  int layers, hidden, q_heads, kv_heads, head_dim, inter, vocab, max_ctx;   // this rank's (local) sizes
  float rms_eps;
  int k_blocked = 0;                  // K caches block-transposed (cai_k_blocked_index); max_ctx is then a multiple of 32
  const QWeight* embed;
  const QWeight* lm_head;
  const float* final_norm;
  const float* theta;                 // [head_dim / 2] RoPE frequencies
  std::vector<StepLayerSetup> layer;
  int32_t *tokens, *pos, *len;        // device words of the session (one sequence)
  float *xres, *qbuf, *att, *act, *logits, *partial;
  size_t partial_floats;              // capacity of `partial`
  int32_t* amax_idx; float* amax_val;
  int32_t* trace; int32_t* trace_count; int64_t trace_cap;
  // tensor parallel (world > 1): the peer-memory exchange the step kernel uses for its sums over the ranks
  cai_tp_ar* ar = nullptr;
  int tp_rank = 0, tp_world = 1;
  int vocab_offset = 0;               // first vocabulary row of this rank's LM-head shard
};

struct StepPlan;
// CAI_ERR_UNSUPPORTED (and *out == NULL) when the model or session is outside what the kernel covers; the caller
// then keeps the launch-per-operator path.
int step_plan_create(cai_ctx* ctx, const StepSetup& s, StepPlan** out);
void step_plan_destroy(StepPlan* p);
// Enqueues one decode step on the context's stream. ts_dev (nullable): device array of at least
// step_plan_trace_len() 64-bit words that receives the global-timer value at every phase boundary.
int step_plan_enqueue(cai_ctx* ctx, StepPlan* p, unsigned long long* ts_dev);
int step_plan_trace_len(const StepPlan* p);
// family (FAM_*) of the phase that ENDS at trace entry i (entry 0 is the kernel's start)
int step_plan_trace_family(const StepPlan* p, int i);
// Clears the barrier words after a step that gave up a wait.
int step_plan_reset_sync(cai_ctx* ctx, StepPlan* p);

// comm.cu: what the step kernel needs from the peer-memory exchange
struct TpExchange {
  int rank, world;
  int* my_flags;                 // [world] arrival words of this rank (peers write theirs)
  int* peer_flags[8];            // every rank's arrival words
  float* my_slots;               // [sites][max_elems] partial results of this rank
  const float* peer_slots[8];    // every rank's slots
  int64_t max_elems;
  int sites;
  int* seq;                      // device word: exchanges completed so far
  int* gave_up;                  // device word: a wait of this rank ran out
};
int comm_ar_exchange(cai_tp_ar* ar, TpExchange* out);
