/*
 * cai_cuda.h - C ABI of the B200 (sm_100a) decode backend for CAI Neural API.
 *
 * A cdecl shared library (libcai_cuda.so) that a Free Pascal unit placed beside
 * neural/neuralopencl.pas binds with `external 'cai_cuda'` declarations. Plain
 * C types only: no C++ types, no PyTorch types. Every entry point returns an
 * int status (CAI_OK == 0) and never throws; the message of the last failure is
 * read with cai_cuda_last_error, the way the OpenCL backend reports cl_int
 * results through ErrorProc callbacks (neural/neuralopencl.pas:740-753,
 * 1051-1055).
 *
 * Threading: one caller thread per context, like the reference's shared
 * in-order queue that funnels every device layer through scheduler worker 0
 * (examples/ChatTerminal/README.md:174-180). Work is enqueued on one CUDA
 * stream owned by the context.
 *
 * Pointers named *_host are host memory owned by the caller; pointers named
 * *_dev are device memory on the context's GPU (from cai_dev_alloc or another
 * entry point of this library).
 */
#ifndef CAI_CUDA_H
#define CAI_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cai_ctx cai_ctx;
typedef struct cai_linear cai_linear;
typedef struct cai_sdpa cai_sdpa;
typedef struct cai_model cai_model;
typedef struct cai_session cai_session;

/* status codes */
enum {
  CAI_OK = 0,
  CAI_ERR_INVALID = 1,      /* bad argument, shape or handle */
  CAI_ERR_CUDA = 2,         /* a CUDA runtime call failed */
  CAI_ERR_OOM = 3,          /* device allocation failed or request too large */
  CAI_ERR_STATE = 4,        /* call out of order (e.g. step before finalize, context full) */
  CAI_ERR_UNSUPPORTED = 5,  /* tensor type or shape outside what the kernels cover */
  CAI_ERR_COMM = 6          /* multi-GPU communicator failure */
};

/* Tensor storage types: the ggml type ids a GGUF file carries
 * (neural/neuralgguf.pas:100-131). */
enum {
  CAI_TYPE_F32 = 0,
  CAI_TYPE_F16 = 1,
  CAI_TYPE_Q4_0 = 2,  /* 18-byte blocks of 32: fp16 d, 16 nibble bytes; x = d*(nib-8)  (neuralgguf.pas:822-845) */
  CAI_TYPE_Q8_0 = 8,  /* 34-byte blocks of 32: fp16 d, 32 int8;          x = d*q        (neuralgguf.pas:1487-1503) */
  /* K-quants that stay resident as the file's raw super-blocks of 256 (rows are whole super-blocks, K % 256 == 0) and run
     on their own dequant-fused GEMV. The resident blocks dequantize exactly as the reference's decoders do
     (DequantizeQ4K / Q5K / Q6K, neuralgguf.pas:474-738: cai_linear_dequantize, cai_model_read_tensor); the product
     regroups a run's arithmetic as dl * sum(code * x) - ml * sum(x) with dl = d * sc and ml = dmin * mn rounded as the
     decoder rounds them, the way the Q8_0 / Q4_0 kernels apply a block scale to a sum. Batches run in groups of up to
     4 rows per pass. */
  CAI_TYPE_Q4_K = 12, /* 144-byte super-blocks */
  CAI_TYPE_Q5_K = 13, /* 176-byte super-blocks */
  CAI_TYPE_Q6_K = 14, /* 210-byte super-blocks */
  /* Load-time formats: accepted by cai_model_upload_tensor, cai_linear_create, cai_dequantize and the GGUF loader; decoded
     on the device to fp32 when they arrive, as the reference's reader does (DecodeGGMLSpan, neuralgguf.pas:1471-1523), and
     resident as F32 (or as CAI_TYPE_I8ROW under cai_model_set_int8_weights). Block rules: neuralgguf.pas:448-945. */
  CAI_TYPE_Q4_1 = 3,  /* 20-byte blocks of 32 */
  CAI_TYPE_Q5_0 = 6,  /* 22-byte blocks of 32 */
  CAI_TYPE_Q5_1 = 7,  /* 24-byte blocks of 32 */
  CAI_TYPE_Q2_K = 10, /* 84-byte super-blocks of 256 */
  CAI_TYPE_Q3_K = 11, /* 110-byte super-blocks of 256 */
  CAI_TYPE_I8ROW = 124, /* the reference's own int8 weights (what ChatTerminal runs by default): int8 codes [N][K] and ONE fp32
                         scale per output row, scale = maxabs/127, code = Round(v * (1/maxabs) * 127) with round-half-to-even
                         (TNNetVolume.QuantizeInt8 / MaxAbsFinite, neural/neuralvolume.pas:12471-12562); the product is the raw
                         sum of code * x in fp32 with the row scale applied once after the sum (DotProductsTiledInt8,
                         :12693-12745). Not a ggml id. Host row format of this library: K code bytes followed by the row's
                         4-byte scale; K % 16 == 0 */
  CAI_TYPE_I8 = 24    /* KV cache only: int8 codes + one fp32 scale per (head, position) row, scale = maxabs/127
                         (neural/neural.cl:2500-2687, TNNetFusedSDPA.BeginIncrementalDecode(MaxCtx, Int8KV = true)) */
};

/* Activation opcodes of the fused linear epilogue; the numbering of
 * cai_dot_product_int8 (neural/neural.cl:161-291): 0 none, 1 ReLU, 2 sigmoid, 3 tanh. */
enum { CAI_ACT_NONE = 0, CAI_ACT_RELU = 1, CAI_ACT_SIGMOID = 2, CAI_ACT_TANH = 3 };

/* ------------------------------------------------------------------------- */
/* Context. Replaces TEasyOpenCL platform/device/queue setup                  */
/* (neural/neuralopencl.pas:72-164) and the TNNet.EnableOpenCL hook           */
/* (neural/neuralchatengine.pas:1156-1157).                                   */
/* ------------------------------------------------------------------------- */
int cai_cuda_init(int device_id, cai_ctx** out_ctx);
int cai_cuda_shutdown(cai_ctx* ctx);
/* Copies the last error message of this context (NUL terminated) into buf. */
int cai_cuda_last_error(cai_ctx* ctx, char* buf, int buf_len);
/* sm_count, total device bytes; either pointer may be NULL. */
int cai_cuda_device_info(cai_ctx* ctx, int* sm_count, int64_t* total_bytes);
/* Number of kernels this library has launched on the context since init. */
int cai_cuda_launch_count(cai_ctx* ctx, int64_t* out_count);
/* 1 when this library is the checked build (libcai_cuda_checked.so, compiled with -DCAI_CHECKED): the same kernels,
 * every launch followed by a synchronize and a look at the device error words, CUDA graphs off, and an index from
 * device-side state that the ordinary build clamps or skips silently (an out-of-range token id, an expert id outside
 * the bank) reported as CAI_ERR_STATE with its value and bound. 0 for the ordinary build. Needs no context.
 * No reference counterpart. */
int cai_cuda_is_checked_build(void);

/* Longest time a kernel of this library waits on another CTA or another GPU (grid barrier of the step kernel,
 * arrival words of the tensor-parallel exchange) before it gives up, raises the context's error word and returns;
 * the next synchronizing entry point then reports CAI_ERR_CUDA and the context stays usable. Default 2 s
 * (environment CAI_WAIT_LIMIT_US). No reference counterpart: the OpenCL backend has no device-side waits. */
int cai_cuda_set_wait_limit_us(cai_ctx* ctx, unsigned limit_us);
/* Failure-path self-test: makes one such wait run out on purpose (no peer needed, nothing hangs).
 * which = 0: the all-reduce kernel waiting for a rank that does not exist; 1: the step kernel's grid barrier with one
 * arrival missing. Returns CAI_ERR_CUDA when the time-out path worked as designed. No reference counterpart. */
int cai_selftest_wait_timeout(cai_ctx* ctx, int which, unsigned limit_us);

/* Device buffers: the cl_mem create/write/read calls of TEasyOpenCLV
 * (neural/neuralopencl.pas:167-202). */
int cai_dev_alloc(cai_ctx* ctx, int64_t bytes, void** out_dev);
int cai_dev_free(cai_ctx* ctx, void* dev);
int cai_memcpy_h2d(cai_ctx* ctx, void* dst_dev, const void* src_host, int64_t bytes);
int cai_memcpy_d2h(cai_ctx* ctx, void* dst_host, const void* src_dev, int64_t bytes);
int cai_dev_sync(cai_ctx* ctx);
/* Device-time bracket on the context's stream (CUDA events):
 * begin records, end records, synchronizes and returns the milliseconds. */
int cai_timer_begin(cai_ctx* ctx);
int cai_timer_end(cai_ctx* ctx, float* out_ms);
/* Overwrites a private device buffer larger than the L2 cache (cold-cache timing). */
int cai_flush_l2(cai_ctx* ctx);

/* ------------------------------------------------------------------------- */
/* Block codec check hook: dequantizes on the GPU through the same resident   */
/* layout the linear kernels read, so the result must be bit-identical to     */
/* DecodeGGMLSpan (neural/neuralgguf.pas:1471-1523).                          */
/* ------------------------------------------------------------------------- */
int cai_dequantize(cai_ctx* ctx, int type, const void* blocks_host, int64_t rows, int64_t cols,
                   float* out_host);

/* ------------------------------------------------------------------------- */
/* Quantized linear layer. Replaces TDotProductSharedKernel                   */
/* (neural/neuralopencl.pas:245-388):                                         */
/*   cai_linear_create       <- PrepareForComputeInt8 (:844-891): weights are */
/*                              uploaded ONCE and stay resident and immutable */
/*   cai_linear_forward      <- ComputeInt8 + FinishAndLoadResult (:946-1104) */
/*                              with host operands (NewVBs = true)            */
/*   cai_linear_forward_dev  <- ComputeInt8 with pExternalVBs / ResultBuffer  */
/*                              (:352-356, 382-387): operands stay on device  */
/* Weights are [N rows, K cols] row-major in `type` blocks (K % 32 == 0 for   */
/* Q8_0/Q4_0), output layout y[b*N + a] (neural/neuralvolume.pas:12736).      */
/* ------------------------------------------------------------------------- */
int cai_linear_create(cai_ctx* ctx, int type, const void* blocks_host, int64_t n_rows, int64_t k_cols,
                      const float* bias_host /* nullable, N floats */, cai_linear** out);
/* The same layer from the reference's int8 container (GetInt8QuantData: Codes[n*K + i], Scales[n],
 * tests/TestNeuralPretrained.pas:7004-7016), i.e. TDotProductSharedKernel.PrepareForComputeInt8
 * (neural/neuralopencl.pas:844-891) without re-quantizing anything. K % 16 == 0. */
int cai_linear_create_int8(cai_ctx* ctx, const int8_t* codes_host, const float* scales_host, int64_t n_rows, int64_t k_cols,
                           const float* bias_host /* nullable */, cai_linear** out);
/* QuantizeInt8 + MaxAbsFinite on the device for `rows` rows of `cols` floats (neural/neuralvolume.pas:12471-12562):
 * codes_out_host[rows*cols], scales_out_host[rows] (scale = maxabs/127; 0 for an all-zero row). */
int cai_quantize_int8_rows(cai_ctx* ctx, const float* w_host, int64_t rows, int64_t cols, int8_t* codes_out_host, float* scales_out_host);
int cai_linear_destroy(cai_linear* lin);
int cai_linear_forward(cai_linear* lin, const float* x_host, int batch, float* y_host, int act);
int cai_linear_forward_dev(cai_linear* lin, const float* x_dev, int batch, float* y_dev, int act);
/* Enqueues iters passes over `count` resident layers of identical shape (same x, same y), without
 * returning to the caller between launches: the measurement loop for kernels shorter than a host call. */
int cai_linear_forward_many(cai_linear* const* lins, int count, const float* x_dev, int batch, float* y_dev, int iters);
/* Resident weight bytes (codes + scales), the algorithmic bytes one forward streams. */
int cai_linear_weight_bytes(cai_linear* lin, int64_t* out_bytes);
/* Dequantizes the RESIDENT (repacked) weights to fp32 [N*K] on the host. */
int cai_linear_dequantize(cai_linear* lin, float* out_host);
/* Forces one kernel family for cai_linear_forward*: 0 auto, 1 CUDA-core GEMV, 2 tcgen05 GEMM. */
int cai_linear_set_path(cai_linear* lin, int path);

/* ------------------------------------------------------------------------- */
/* Layer-granular shims on device buffers (a TNNetLayer.ComputeCUDA override  */
/* delegates one layer at a time, like ComputeOpenCL). Token rows are         */
/* depth-contiguous: x[t*depth + c] (neural/neuralvolume.pas:8951-8954).      */
/* ------------------------------------------------------------------------- */
/* cai_token_norm with FUseMean = 0 (neural/neural.cl:1047-1085). y may alias x. */
int cai_rmsnorm_dev(cai_ctx* ctx, const float* x_dev, const float* gain_dev, float* y_dev,
                    int tokens, int depth, float eps);
/* cai_rope (neural/neural.cl:1517-1542): pairs (2k,2k+1), head-tiled theta_k =
 * base^(-2k/head_dim), token t rotates by (t + position_offset). In place. */
int cai_rope_dev(cai_ctx* ctx, float* x_dev, int tokens, int depth, int head_dim,
                 int position_offset, float theta_base);
/* cai_glu_gate with FActFlag = 1 (neural/neural.cl:1213-1263):
 * y[t*half + d] = x[t*2half + d] * swish(x[t*2half + half + d]). */
int cai_swiglu_dev(cai_ctx* ctx, const float* x_dev, float* y_dev, int tokens, int half_depth);
/* softmax -> top-k -> optional renormalisation of one router row per token
 * (TNNetPointwiseSoftMax + TNNetTopKGate, neural/neuralpretrained.pas:15347-15366).
 * Writes k expert ids and k gate values per token; ties: lowest index wins. */
int cai_topk_gate_dev(cai_ctx* ctx, const float* router_logits_dev, int tokens, int n_experts,
                      int top_k, int renorm, int32_t* expert_ids_dev, float* gates_dev);

/* Mixture-of-experts expert bank, layer at a time: TNNetMoEExpertBankGateUp(E, I, ...) and TNNetMoEExpertBankDown(E, H)
 * (wiring neural/neuralpretrained.pas:15347-15388; device twin of the down bank cai_moe_expert_down,
 * neural/neural.cl:2709-2807; semantics tests/TestNeuralLayersExtra.pas:7773-7906). The bank holds, per expert, the up and
 * gate matrices [expert_width, hidden] and the down matrix [hidden, expert_width] in one storage type (F32, F16, Q8_0,
 * Q4_0), bias-free. Slots: token t's j-th selected expert is slot_expert[t*top_k + j] with gate slot_gate[t*top_k + j]
 * (what cai_topk_gate_dev writes); every token fills all top_k slots.
 *   cai_moe_gate_up_dev: hidden_out[(t*top_k + j)*expert_width + d] = up_e(x_t)[d] * swish(gate_e(x_t)[d])
 *   cai_moe_down_dev:    out[t*hidden + h] = sum over j, in slot order, of slot_gate * down_e(hidden_(t,j))[h]
 * which = 0 up, 1 gate, 2 down in cai_moe_bank_upload; blocks are rows in `type` blocks along the input width. */
typedef struct cai_moe_bank cai_moe_bank;
int cai_moe_bank_create(cai_ctx* ctx, int n_experts, int hidden, int expert_width, int type, cai_moe_bank** out);
int cai_moe_bank_destroy(cai_moe_bank* b);
int cai_moe_bank_upload(cai_moe_bank* b, int expert, int which, const void* blocks_host);
int cai_moe_bank_finalize(cai_moe_bank* b);
int cai_moe_gate_up_dev(cai_moe_bank* b, const float* x_dev, const int32_t* slot_expert_dev, int tokens, int top_k,
                        float* hidden_out_dev);
int cai_moe_down_dev(cai_moe_bank* b, const float* hidden_dev, const int32_t* slot_expert_dev, const float* slot_gate_dev,
                     int tokens, int top_k, float* out_dev);

/* Fused GQA attention with a KV cache: TNNetFusedSDPA in incremental-decode mode
 * (BeginIncrementalDecode / ResetCache / TruncateCache / CacheLength,
 * tests/TestNeuralFusedSDPA.pas:226-236, 329-420; kernels neural/neural.cl:2354-2379,
 * 2406-2499). Input row packing [allQ | allK | allV]; cache head-major. */
int cai_sdpa_create(cai_ctx* ctx, int q_heads, int kv_heads, int head_dim, int max_ctx, cai_sdpa** out);
int cai_sdpa_destroy(cai_sdpa* s);
int cai_sdpa_reset(cai_sdpa* s);
int cai_sdpa_truncate(cai_sdpa* s, int committed_len);
int cai_sdpa_cache_len(cai_sdpa* s, int* out_len);
/* The layer's Window and EnableEviction (see cai_session_set_window / cai_session_enable_eviction). */
int cai_sdpa_set_window(cai_sdpa* s, int window);
int cai_sdpa_enable_eviction(cai_sdpa* s, int sink_tokens, int recent_window);
/* Appends the row's K,V at slot CacheLength, then attends the row's Q over the
 * whole cache. out_dev: q_heads*head_dim floats. */
int cai_sdpa_step_dev(cai_sdpa* s, const float* qkv_row_dev, float* out_dev);

/* Allocation-free variant of cai_sdpa_step_dev. It has no counterpart in the reference.
 * For callers that must not allocate device memory when they call in: real-time loops that cannot
 * block in the driver's allocator, plugins confined to an arena their host application handed them,
 * processes whose device-memory budget was fixed at start-up. The caller owns every buffer: the token row
 * [allQ | allK | allV], the head-major K and V caches ([kv_head][max_ctx][head_dim] floats each), one
 * device int holding the number of rows already cached (the caller adds 1 after the call), and the
 * output (q_heads*head_dim floats). The split-context partial results go to a fixed 2 MiB array that is
 * part of the library (each GPU that loads the library holds it until the process exits); a shape whose
 * partials need more (q_heads x context splits x (head_dim+2) floats > 524288) is rejected with
 * CAI_ERR_UNSUPPORTED. The call performs no cudaMalloc / cudaFree and launches on the context's stream
 * without synchronizing. Its first call on a device looks up the array's device address; make that
 * first call before any stream capture. All calls share the array: two calls that overlap on the GPU
 * (different streams, different contexts on one device) race; nothing in it needs clearing between calls.
 * Precondition: 0 <= *cache_len_dev < max_ctx (there must be room for the row this call appends). The host
 * cannot see that word, so the kernels check it: outside the range they touch neither cache nor output and raise
 * the context's error word, which cai_dev_sync then reports as CAI_ERR_STATE. */
int cai_sdpa_step_noalloc(cai_ctx* ctx, float* qkv_row_dev, float* k_cache_dev, float* v_cache_dev,
                          const int32_t* cache_len_dev, int q_heads, int kv_heads, int head_dim, int max_ctx,
                          float* out_dev);

/* ------------------------------------------------------------------------- */
/* Whole-model fast path: the graph BuildLlamaFromTensorReaderWithConfig      */
/* wires (neural/neuralpretrained.pas:16196-17473), resident on the GPU.      */
/* ------------------------------------------------------------------------- */
/* Subset of TLlamaConfig (neural/neuralpretrained.pas:677-952). */
typedef struct cai_llama_config {
  int32_t hidden;
  int32_t inter;          /* dense MLP intermediate size (ignored when n_experts > 0) */
  int32_t layers;
  int32_t heads;
  int32_t kv_heads;
  int32_t head_dim;
  int32_t vocab;
  float rms_eps;
  float rope_theta;
  int32_t tie_embeddings; /* LM head = embedding rows (neuralpretrained.pas:15655-15671) */
  int32_t qkv_bias;       /* Qwen2 q/k/v biases (:16960-16965) */
  int32_t qk_norm;        /* OLMoE full-width q/k RMSNorm before RoPE (:16520-16530) */
  int32_t n_experts;      /* 0 = dense */
  int32_t top_k;
  int32_t norm_topk;      /* renormalise the kept router probabilities (:15347-15366) */
  int32_t moe_inter;      /* expert intermediate size */
} cai_llama_config;

/* tp_size > 1 shards attention heads and MLP columns/rows over tp_size processes
 * (one GPU each); ep_size > 1 shards MoE experts. Neither exists in the reference. */
int cai_model_create(cai_ctx* ctx, const cai_llama_config* cfg, int tp_rank, int tp_size, cai_model** out);
/* Expert-parallel creation for mixture-of-experts models (no reference counterpart; the reference is single
 * process): dense parts replicated, rank ep_rank keeps experts [ep_rank E / ep_size, (ep_rank + 1) E / ep_size),
 * sessions hold this rank's own sequences. Call cai_comm_init(ctx, ep_rank, ep_size, id) first. Every rank uploads
 * (or generates) the full tensor set; tensors of other ranks' experts are ignored. All ranks must create their
 * sessions with the same batch and step them together. */
int cai_model_create_ep(cai_ctx* ctx, const cai_llama_config* cfg, int ep_rank, int ep_size, cai_model** out_model);
int cai_model_destroy(cai_model* m);
/* One tensor under its HF name ("model.layers.3.self_attn.q_proj.weight", ...) in
 * HF layout: rows = out features, cols = in features, `type` blocks along cols
 * (LoadLlamaLinearWeights, neural/neuralpretrained.pas:14770-14989). 1-D tensors
 * (norm gains, biases) are F32 with rows = 1. interleave_head_dim > 0 applies the
 * importer's q/k row permutation target(h*hd+2k) <- row(h*hd+k),
 * target(h*hd+2k+1) <- row(h*hd+k+hd/2) (:14792-14812); pass 0 for rows already
 * in GGUF order. The host buffer is not retained. With tp_size > 1 the caller
 * passes the FULL tensor and the library keeps this rank's slice. */
int cai_model_upload_tensor(cai_model* m, const char* hf_name, int type, const void* data_host,
                            int64_t rows, int64_t cols, int interleave_head_dim);
/* The importer's pQuantizeInt8 switch (neural/neuralpretrained.pas:14876-14888): when on, every F32 / F16 matrix uploaded
 * afterwards is quantized row by row to CAI_TYPE_I8ROW as it arrives (embedding and LM head included) and the model
 * runs on the int8 kernels. Call before the first upload. */
int cai_model_set_int8_weights(cai_model* m, int on);
/* Fills every tensor on the device: weights N(0, std) from a counter-based
 * generator keyed by (seed, tensor, global element index), quantized to `type`
 * with the GGUF writer's Q8_0 rule (neural/neuralgguf.pas:1950-1993) or ggml's Q4_0
 * rule; norm gains 1; biases N(0, std). Shards generate their own slices. */
int cai_model_init_synthetic(cai_model* m, int type, uint64_t seed, float std);
/* Reads one tensor (this rank's slice) back as GGUF blocks of its storage type.
 * out_bytes_cap guards the host buffer; rows/cols/type of the slice are returned. */
int cai_model_read_tensor(cai_model* m, const char* hf_name, void* out_host, int64_t out_bytes_cap,
                          int* out_type, int64_t* out_rows, int64_t* out_cols);
/* ------------------------------------------------------------------------- */
/* GGUF files on the C side. Replaces TNNetGGUFReader                         */
/* (neural/neuralgguf.pas:168-243; ParseFile :1072-1220; metadata getters     */
/* :1263-1344; LoadTensorFlat :1674+) and the GGUF importers                  */
/* BuildLlamaFromGGUFEx / BuildFromGGUFEx (neural/neuralpretrained.pas:       */
/* 17484-17876). Versions 2 and 3; the reader's checks and refusals follow    */
/* the reference's (bad magic, implausible counts or dimensions, empty or     */
/* duplicate names, nested arrays, rows that are not whole blocks, a data     */
/* range outside the file). A reader needs no GPU; decoding does.             */
/* ------------------------------------------------------------------------- */
typedef struct cai_gguf cai_gguf;
/* err_buf (nullable) receives the reason when the file is refused (CAI_ERR_INVALID). */
int cai_gguf_open(const char* path, cai_gguf** out, char* err_buf, int err_len);
int cai_gguf_close(cai_gguf* g);
int cai_gguf_last_error(cai_gguf* g, char* buf, int buf_len);
/* Any pointer may be NULL. data_start = file offset of the aligned data section. */
int cai_gguf_info(cai_gguf* g, int* version, int* alignment, int64_t* n_meta, int64_t* n_tensors, int64_t* data_start);
/* Metadata. value_type is the GGUF value type id (8 string, 9 array, ...). The getters follow GetMetaInt / GetMetaFloat /
 * GetMetaString: a missing key sets *found = 0 and leaves *out alone (the caller's default stands); a key of another type
 * is CAI_ERR_INVALID. Integers of every width and bools read as int; ints also read as float. */
int cai_gguf_meta_key(cai_gguf* g, int64_t index, char* key_buf, int key_cap, int* value_type);
int cai_gguf_meta_int(cai_gguf* g, const char* key, int64_t* out, int* found);
int cai_gguf_meta_float(cai_gguf* g, const char* key, double* out, int* found);
int cai_gguf_meta_string(cai_gguf* g, const char* key, char* buf, int cap, int* found);
int cai_gguf_meta_array_count(cai_gguf* g, const char* key, int64_t* out_count);   /* 0 when the key is absent */
/* Tensor table. shape8 is in served order, contiguous axis LAST (the stored ggml dims reversed, :1157-1162): a linear
 * weight reads [out, in]. data_begin is relative to the data section; data_bytes is 0 for a type without a decoder. */
int cai_gguf_tensor_info(cai_gguf* g, int64_t index, char* name_buf, int name_cap, int* type, int* ndims, int64_t* shape8,
                         int64_t* data_begin, int64_t* data_bytes);
int cai_gguf_find_tensor(cai_gguf* g, const char* name, int64_t* out_index);       /* -1 when absent */
int cai_gguf_read_raw(cai_gguf* g, int64_t index, void* out_host, int64_t cap_bytes);
/* DecodeGGMLSpan on the device: n_elems elements of `type` blocks (host bytes) -> fp32 (host), bit-identical to the
 * reference's decoders for F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K. */
int cai_gguf_decode(cai_ctx* ctx, int type, const void* raw_host, int64_t n_elems, float* out_host);
/* LoadTensorFlat: tensor `index` decoded to fp32 in flat row-major order. */
int cai_gguf_load_tensor(cai_ctx* ctx, cai_gguf* g, int64_t index, float* out_host, int64_t cap_elems);
/* Metadata -> configuration (architectures llama and qwen2; anything else CAI_ERR_UNSUPPORTED, as are RoPE position
 * interpolation with a factor other than 1 and qwen2 sliding-window files). max_positions (nullable) = <arch>.context_length. */
int cai_gguf_llama_config(cai_gguf* g, cai_llama_config* cfg, int64_t* max_positions);
/* BuildFromGGUFEx: opens the file, builds the configuration, creates the model (this rank's shard when tp_size > 1),
 * uploads every tensor under its HF name and finalizes. q/k rows stay in their stored order, which is the interleaved
 * rotary order the graph runs in (the reference's reader de-interleaves and its loader re-interleaves:
 * neuralgguf.pas:428-438, neuralpretrained.pas:14792-14812). quantize_int8 = the importer's pQuantizeInt8. */
int cai_model_load_gguf(cai_ctx* ctx, const char* path, int tp_rank, int tp_size, int quantize_int8, cai_model** out_model,
                        cai_llama_config* out_cfg /* nullable */, int64_t* out_max_positions /* nullable */);

/* Verifies every tensor the configuration needs is present; required before sessions. */
int cai_model_finalize(cai_model* m);
/* Bytes of matrix weights one decode step streams on this rank (codes + scales). */
int cai_model_step_weight_bytes(cai_model* m, int64_t* out_bytes);

/* Decode session: TNNetStreamingDecoder (neural/neuraldecode.pas:5614-5663 Create,
 * :5686-5694 Reset, :5696-5712 StepForward, :5714-5720 TruncateTo, :5759-5843
 * Snapshot/RestoreSnapshot). `batch` independent sequences step together; the
 * reference has one sequence per session, so per-sequence results must equal the
 * single-sequence path. kv_type: CAI_TYPE_F32 (the --kv-fp32 cache) or CAI_TYPE_I8 (the reference's default
 * int8 cache: rows quantized when appended, scales folded into the attention sums; head_dim 64 or 128, groups of
 * up to 8 query heads per KV head). */
int cai_session_create(cai_model* m, int max_ctx, int batch, int kv_type, cai_session** out);
int cai_session_destroy(cai_session* s);
int cai_session_reset(cai_session* s, int seq /* -1 = all */);
int cai_session_truncate(cai_session* s, int seq, int committed_len);
int cai_session_cache_len(cai_session* s, int seq, int* out_len);
/* TNNetStreamingDecoder.EnableEviction / DisableEviction (neural/neuraldecode.pas:1257-1276, 5722-5727): StreamingLLM.
 * Every layer keeps the first sink_tokens rows and the most recent recent_window rows; a stream then runs forever in
 * a cache of sink_tokens + recent_window rows (<= max_ctx). Keys keep the rotation of their original position and the
 * query its true absolute position, so surviving pairs attend at their exact distance. While a sequence is no longer
 * than sink_tokens + recent_window the output is that of the unbounded session. (0, 0) turns it off. Here the rows
 * live as sinks + a ring instead of being shifted down one by one; the set of live rows is the reference's.
 * cai_session_cache_len keeps counting positions; the rows held are min(len, sink_tokens + recent_window). */
int cai_session_enable_eviction(cai_session* s, int sink_tokens, int recent_window);
/* Sliding-window attention on every layer: a step attends over the most recent `window` cached rows only (the new row
 * included), TNNetFusedSDPA's Window (jStart, neural/neural.cl:2437-2438). 0 = the whole cache. */
int cai_session_set_window(cai_session* s, int window);
/* Benchmark aid, no reference counterpart: zeroes the KV caches and declares n_rows positions cached in every sequence,
 * so that decode steps can be timed at a long context without paying for its prefill (64 sequences x 8192 positions of
 * a 32B model are half a million prefill tokens). The rows are zeros, not the model's: logits of such a session mean
 * nothing, its timing is that of any session with n_rows cached rows. */
int cai_session_fill_for_benchmark(cai_session* s, int n_rows);
/* One width-1 forward per sequence. tokens_host[batch]; abs_pos_host[batch] may be
 * NULL (= cache length, the position StepForward writes into every RoPE layer).
 * logits_out_host (batch*vocab floats) and argmax_out_host (batch ints, first
 * index of the maximum: ArgMaxRow, neural/neuralchatengine.pas:683-697) are
 * nullable. Blocks until the results are on the host. */
int cai_session_step(cai_session* s, const int32_t* tokens_host, const int32_t* abs_pos_host,
                     float* logits_out_host, int32_t* argmax_out_host);
/* Greedy loop kept on the device: feeds tokens_host[batch] then n_steps-1 times
 * the previous argmax (GenerateFromIds decode loop, neural/neuralchatengine.pas:1485-1561,
 * greedy fast path). out_tokens_host[n_steps*batch] (step-major) nullable.
 * No host round trip between steps. */
int cai_session_decode_greedy(cai_session* s, const int32_t* tokens_host, int n_steps,
                              int32_t* out_tokens_host);
/* Sampling without shipping the logits row to the host (the reference's samplers sort 152k scores per token on the
 * CPU, docs/OPTIMIZATION-GUIDE.md:1914-1919).
 * cai_session_step_topk: one step, then the candidate window the reference's samplers work on: the k (<= 64) largest
 * scores of softmax(logits / temperature) over the whole vocabulary, descending, ties to the lower id, as ids and
 * probabilities per sequence (TNNetSamplerBase.SelectTopCandidates, neural/neuralvolume.pas:991-1030, with
 * TNNetTemperatureProcessor applied first). The host's own sampler and random generator then pick: 8 k bytes per
 * sequence come back instead of 4 * vocab.
 * cai_session_decode_sampled: the whole loop on the device. Per step and sequence the draw of
 * TNNetSamplerWeightedTopK.SampleFromSorted (:4749-4785) over that window, optionally cut to the nucleus first (the
 * shortest prefix whose probabilities sum above top_p; top_p <= 0 or >= 1 keeps the window): Roll = u * KeptSum, the
 * first candidate whose running sum exceeds Roll. u comes from uniforms_host[step * batch + seq] when given, else from
 * a counter-based generator keyed by (seed, step counted from 1, sequence) that cai_sampling_uniform reproduces.
 * out_tokens_host[n_steps * batch] nullable. Single-GPU sessions (the vocabulary must not be sharded). */
typedef struct cai_sampling {
  float temperature;   /* > 0; 1 = off */
  int32_t top_k;       /* 1..64 */
  float top_p;         /* nucleus mass; <= 0 or >= 1 = off */
  uint64_t seed;
} cai_sampling;
int cai_session_step_topk(cai_session* s, const int32_t* tokens_host, const int32_t* abs_pos_host, int k, float temperature,
                          int32_t* ids_out_host, float* probs_out_host);
int cai_session_decode_sampled(cai_session* s, const int32_t* tokens_host, int n_steps, const cai_sampling* opt,
                               const float* uniforms_host /* nullable */, int32_t* out_tokens_host);
int cai_sampling_uniform(uint64_t seed, uint64_t step, uint64_t seq, float* out_u);
/* Feeds n_tokens per sequence (tokens_host[seq*n_tokens + i]) one position at a
 * time without reading anything back: the prefill loop of GenerateFromIds
 * (neural/neuralchatengine.pas:1466-1470). */
int cai_session_prefill(cai_session* s, const int32_t* tokens_host, int n_tokens);
/* Per-launch device timing of n_steps eager (non-graph) steps fed like cai_session_decode_greedy:
 * one CUDA event after every launch on the context's stream, times summed per kernel family.
 * out_ms[4] / out_launches[4]: 0 linear layers, 1 attention, 2 other operators, 3 collectives.
 * The per-layer-class report of TNNet.LayerClassTimingReport (neural/neuralchatengine.pas:1613-1623).
 * Advances the session by n_steps. */
int cai_session_profile(cai_session* s, const int32_t* tokens_host, int n_steps, float* out_ms, int64_t* out_launches);
/* Deep copy of the KV caches and lengths / restore (TNNetDecoderSessionSnapshot). */
int cai_session_snapshot(cai_session* s);
int cai_session_restore(cai_session* s);
/* Device logits of the last step, [batch*vocab] (this rank's shard when tp_size > 1). */
int cai_session_logits_dev(cai_session* s, const float** out_dev);
/* One cached K row and V row of (layer, sequence, KV head, position), whatever the internal cache layout: the
 * check hook that TNNetFusedSDPA's CaptureCacheState / the FKCache, FKCacheCodes, FKCacheScale fields give the
 * reference's tests (tests/TestNeuralFusedSDPA.pas:329-420). fp32 cache: head_dim floats into k_out_host / v_out_host
 * (the code and scale outputs may be NULL). int8 cache: head_dim codes into k_codes_host / v_codes_host, the two row
 * scales into scales_host[0..1], and, when given, code * scale into k_out_host / v_out_host. */
int cai_session_read_kv_row(cai_session* s, int layer, int seq, int kv_head, int pos, float* k_out_host, float* v_out_host,
                            int8_t* k_codes_host, int8_t* v_codes_host, float* scales_host);
/* 1 when the session runs each step as ONE persistent kernel (dense model, one sequence, Q8_0 weights, fp32 cache,
 * head_dim 64 or 128; environment CAI_STEP_KERNEL=0 turns it off), 0 when it enqueues one kernel per operator the way
 * the reference enqueues one OpenCL kernel per layer (neural/neuralopencl.pas:946-1056). */
int cai_session_uses_step_kernel(cai_session* s, int* out_flag);
/* One decode step of a step-kernel session with the phase trace switched on: CTA 0 stamps the GPU's global timer
 * when it leaves each grid barrier. out_ns[k] = nanoseconds since the kernel's first stamp, out_family[k] = what ended
 * there (0 a matrix product, 1 attention or the merge of its splits, 2 anything else, 3 an exchange between GPUs);
 * *out_n entries, at most cap. Feeds tokens_host[1] like cai_session_step and advances the session by one position.
 * The finer-grained sibling of cai_session_profile. */
int cai_session_step_trace(cai_session* s, const int32_t* tokens_host, int64_t* out_ns, int32_t* out_family, int cap, int* out_n);
/* Bytes of KV cache the last step read (for the roofline arithmetic). */
int cai_session_last_kv_bytes(cai_session* s, int64_t* out_bytes);

/* ------------------------------------------------------------------------- */
/* Multi-GPU plumbing (no reference counterpart): one process per GPU. The    */
/* 128-byte id is created on rank 0 and handed to the others by the host      */
/* program (torch.distributed, MPI, a file ...).                              */
/* ------------------------------------------------------------------------- */
int cai_comm_unique_id(unsigned char out_id[128]);
int cai_comm_init(cai_ctx* ctx, int rank, int world, const unsigned char id[128]);
int cai_comm_allreduce_dev(cai_ctx* ctx, float* buf_dev, int64_t count);

#ifdef __cplusplus
}
#endif
#endif /* CAI_CUDA_H */
