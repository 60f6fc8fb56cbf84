// Whole-model fast path: the Llama-family graph resident on the GPU and the
// decode session that steps it one token per sequence over a KV cache.
//
// Weight conventions follow the reference importer: nn.Linear rows = output
// channels, q/k rows interleaved per head for the pairwise RoPE, fused gate|up
// matrix with the up rows first and the gate rows second, experts laid out the
// same way per expert.
#include "cai_common.cuh"
#include "step_kernel.cuh"
#include <new>
#include <math.h>
#include <stdlib.h>

enum TKind {
  T_EMBED, T_LM_HEAD, T_FINAL_NORM, T_ATTN_NORM, T_FFN_NORM, T_Q, T_K, T_V, T_QB, T_KB, T_VB, T_O,
  T_GATE, T_UP, T_DOWN, T_QNORM, T_KNORM, T_ROUTER, T_EXP_GATE, T_EXP_UP, T_EXP_DOWN, T_IGNORE, T_UNKNOWN
};
struct TName { TKind kind; int layer; int expert; };

static TName parse_name(const char* name) {
  TName t{T_UNKNOWN, -1, -1};
  if (!strcmp(name, "model.embed_tokens.weight")) { t.kind = T_EMBED; return t; }
  if (!strcmp(name, "lm_head.weight")) { t.kind = T_LM_HEAD; return t; }
  if (!strcmp(name, "model.norm.weight")) { t.kind = T_FINAL_NORM; return t; }
  int layer = -1, consumed = 0;
  if (sscanf(name, "model.layers.%d.%n", &layer, &consumed) < 1 || consumed == 0) return t;
  t.layer = layer;
  const char* rest = name + consumed;
  struct { const char* s; TKind k; } simple[] = {
      {"input_layernorm.weight", T_ATTN_NORM}, {"post_attention_layernorm.weight", T_FFN_NORM},
      {"self_attn.q_proj.weight", T_Q}, {"self_attn.k_proj.weight", T_K}, {"self_attn.v_proj.weight", T_V},
      {"self_attn.q_proj.bias", T_QB}, {"self_attn.k_proj.bias", T_KB}, {"self_attn.v_proj.bias", T_VB},
      {"self_attn.o_proj.weight", T_O}, {"mlp.gate_proj.weight", T_GATE}, {"mlp.up_proj.weight", T_UP},
      {"mlp.down_proj.weight", T_DOWN}, {"self_attn.q_norm.weight", T_QNORM}, {"self_attn.k_norm.weight", T_KNORM},
      {"mlp.gate.weight", T_ROUTER}, {"block_sparse_moe.gate.weight", T_ROUTER},
      {"self_attn.rotary_emb.inv_freq", T_IGNORE}};
  for (auto& e : simple) if (!strcmp(rest, e.s)) { t.kind = e.k; return t; }
  int ex = -1; consumed = 0;
  const char* er = nullptr;
  if (sscanf(rest, "mlp.experts.%d.%n", &ex, &consumed) >= 1 && consumed) er = rest + consumed;
  else { consumed = 0; if (sscanf(rest, "block_sparse_moe.experts.%d.%n", &ex, &consumed) >= 1 && consumed) er = rest + consumed; }
  if (er) {
    t.expert = ex;
    if (!strcmp(er, "gate_proj.weight") || !strcmp(er, "w1.weight")) t.kind = T_EXP_GATE;
    else if (!strcmp(er, "up_proj.weight") || !strcmp(er, "w3.weight")) t.kind = T_EXP_UP;
    else if (!strcmp(er, "down_proj.weight") || !strcmp(er, "w2.weight")) t.kind = T_EXP_DOWN;
  }
  return t;
}

enum {
  HAVE_ATTN_NORM = 1, HAVE_FFN_NORM = 2, HAVE_Q = 4, HAVE_K = 8, HAVE_V = 16, HAVE_QB = 32, HAVE_KB = 64, HAVE_VB = 128,
  HAVE_O = 256, HAVE_GATE = 512, HAVE_UP = 1024, HAVE_DOWN = 2048, HAVE_QNORM = 4096, HAVE_KNORM = 8192, HAVE_ROUTER = 16384
};

struct LayerW {
  float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  float* qkv_bias = nullptr;                  // [q | k | v] biases, owned here; wqkv.bias aliases it after finalize
  QWeight wqkv, wo, wgu, wdown, router;
  // A file may store the members of a fused matrix in different formats (llama.cpp's mixed K-quant presets: q and k in
  // Q4_K, v in Q6_K). Such a group is kept as separate matrices, each in its own format, and the step runs one product
  // per member with the plain epilogue (RoPE + append and SwiGLU then run as their own kernels).
  QWeight wq_part[3];                         // q, k, v when qkv_split
  QWeight wgu_part[2];                        // up, gate when gu_split
  bool qkv_split = false, gu_split = false;
  std::vector<QWeight> exp_gu, exp_down;
  std::vector<uint8_t> exp_have;              // bit 1 gate, 2 up, 4 down
  const void** d_gu_codes = nullptr; const __half** d_gu_scales = nullptr;
  const void** d_down_codes = nullptr; const __half** d_down_scales = nullptr;
  uint32_t have = 0;
};

struct cai_model {
  cai_ctx* ctx;
  cai_llama_config cfg;
  int tp_rank, tp_size;
  // expert parallelism (cai_model_create_ep): the dense parts are replicated, rank r owns experts
  // [r * n_experts / ep_size, (r + 1) * n_experts / ep_size); sessions hold this rank's share of the sequences
  int ep_rank = 0, ep_size = 1;
  int expert_lo() const { return ep_rank * (cfg.n_experts / ep_size); }
  int expert_hi() const { return (ep_rank + 1) * (cfg.n_experts / ep_size); }
  bool owns_expert(int e) const { return e >= expert_lo() && e < expert_hi(); }
  // local (this rank's) dimensions
  int heads_l, kv_heads_l, qw_l, kw_l, inter_l, vocab_l;
  QWeight embed, lm_head;
  bool have_embed = false, have_head = false;
  float* final_norm = nullptr;
  float* theta = nullptr;
  std::vector<LayerW> layers;
  bool finalized = false;
  int sessions = 0;
  bool int8_weights = false;     // quantize F32 matrices to int8 rows as they are uploaded (the importer's pQuantizeInt8)
};

static int ensure_weight(cai_ctx* ctx, QWeight* w, int type, int64_t n, int64_t k) {
  if (w->codes) {
    if (w->type != type || w->n != n || w->k != k)
      return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "tensors fused into one matrix must share one storage type (have %d, got %d)", w->type, type);
    return CAI_OK;
  }
  return qweight_alloc(ctx, w, type, n, k);
}
// Moves the members of a fused matrix that were uploaded so far into matrices of their own (same type, planes copied
// on the device) and frees the fused one: the group continues in split form.
static int split_fused(cai_ctx* ctx, QWeight* fused, QWeight* parts, const int64_t* row0, const int64_t* nrows, const bool* have, int n_parts) {
  for (int i = 0; i < n_parts; ++i) {
    if (!have[i]) continue;
    const QWeight v = qweight_rows_view(*fused, row0[i], nrows[i]);
    CAI_TRY(qweight_alloc(ctx, &parts[i], fused->type, nrows[i], fused->k));
    CAI_CUDA(ctx, cudaMemcpyAsync(parts[i].codes, v.codes, parts[i].code_bytes(), cudaMemcpyDeviceToDevice, ctx->stream));
    if (v.scales) CAI_CUDA(ctx, cudaMemcpyAsync(parts[i].scales, v.scales, parts[i].scale_alloc_bytes(), cudaMemcpyDeviceToDevice, ctx->stream));
    if (v.rscale) CAI_CUDA(ctx, cudaMemcpyAsync(parts[i].rscale, v.rscale, (size_t)nrows[i] * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    parts[i].present = true;
  }
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  fused->bias = nullptr;
  qweight_free(fused);
  return CAI_OK;
}
static int ensure_vec(cai_ctx* ctx, float** p, int64_t n, bool zero) {
  if (*p) return CAI_OK;
  CAI_CUDA(ctx, cudaMalloc((void**)p, (size_t)n * 4));
  if (zero) CAI_CUDA(ctx, cudaMemsetAsync(*p, 0, (size_t)n * 4, ctx->stream));
  return CAI_OK;
}
// host vector slice [g0, g0+n) of a length-`total` fp32 vector, optional per-head interleave, to device
static int upload_vec(cai_ctx* ctx, float* dst, const float* host, int64_t total, int64_t g0, int64_t n, int interleave_hd) {
  std::vector<float> tmp((size_t)n);
  for (int64_t i = 0; i < n; ++i) {
    int64_t g = g0 + i;
    if (interleave_hd > 0) {
      const int64_t h = g / interleave_hd, r = g % interleave_hd;
      g = h * interleave_hd + ((r % 2 == 0) ? r / 2 : r / 2 + interleave_hd / 2);
    }
    if (g >= total) return cai_fail(ctx, CAI_ERR_INVALID, "vector index out of range");
    tmp[(size_t)i] = host[g];
  }
  CAI_CUDA(ctx, cudaMemcpyAsync(dst, tmp.data(), (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

static void layer_free(LayerW& L) {
  if (L.attn_norm) cudaFree(L.attn_norm);
  if (L.ffn_norm) cudaFree(L.ffn_norm);
  if (L.q_norm) cudaFree(L.q_norm);
  if (L.k_norm) cudaFree(L.k_norm);
  if (L.qkv_bias) cudaFree(L.qkv_bias);
  L.wqkv.bias = nullptr;
  for (auto& w : L.wq_part) { w.bias = nullptr; qweight_free(&w); }
  for (auto& w : L.wgu_part) qweight_free(&w);
  qweight_free(&L.wqkv); qweight_free(&L.wo); qweight_free(&L.wgu); qweight_free(&L.wdown); qweight_free(&L.router);
  for (auto& w : L.exp_gu) qweight_free(&w);
  for (auto& w : L.exp_down) qweight_free(&w);
  if (L.d_gu_codes) cudaFree((void*)L.d_gu_codes);
  if (L.d_gu_scales) cudaFree((void*)L.d_gu_scales);
  if (L.d_down_codes) cudaFree((void*)L.d_down_codes);
  if (L.d_down_scales) cudaFree((void*)L.d_down_scales);
}

extern "C" {

int cai_model_create(cai_ctx* ctx, const cai_llama_config* cfg, int tp_rank, int tp_size, cai_model** out) {
  CAI_TRY(cai_bind(ctx));
  if (!cfg || !out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_create: null argument");
  *out = nullptr;
  const cai_llama_config& c = *cfg;
  if (c.hidden < 1 || c.layers < 1 || c.heads < 1 || c.kv_heads < 1 || c.head_dim < 2 || (c.head_dim % 2) || c.vocab < 1 ||
      (c.heads % c.kv_heads) || (c.n_experts == 0 && c.inter < 1) || c.head_dim > 256)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_create: inconsistent configuration");
  if (c.n_experts > 0 && (c.top_k < 1 || c.top_k > c.n_experts || c.moe_inter < 1))
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_create: inconsistent MoE configuration");
  if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return cai_fail(ctx, CAI_ERR_INVALID, "tp rank %d of %d", tp_rank, tp_size);
  if (tp_size > 1) {
    if (c.n_experts > 0 || c.qk_norm) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "tensor parallelism covers dense models without full-width q/k norm");
    if ((c.heads % tp_size) || (c.kv_heads % tp_size) || (c.inter % tp_size) || (c.vocab % tp_size) || ((c.inter / tp_size) % 32) ||
        ((c.heads / tp_size * c.head_dim) % 32))
      return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "heads/kv_heads/inter/vocab must divide by tp_size with 32-aligned shards");
    if (comm_world(ctx) != tp_size) return cai_fail(ctx, CAI_ERR_STATE, "call cai_comm_init with world == tp_size first");
  }
  cai_model* m = new (std::nothrow) cai_model();
  if (!m) return cai_fail(ctx, CAI_ERR_OOM, "host allocation failed");
  m->ctx = ctx; m->cfg = c; m->tp_rank = tp_rank; m->tp_size = tp_size;
  m->heads_l = c.heads / tp_size; m->kv_heads_l = c.kv_heads / tp_size;
  m->qw_l = m->heads_l * c.head_dim; m->kw_l = m->kv_heads_l * c.head_dim;
  m->inter_l = c.n_experts ? 0 : c.inter / tp_size;
  m->vocab_l = c.vocab / tp_size;
  m->layers.resize((size_t)c.layers);
  if (c.n_experts)
    for (auto& L : m->layers) { L.exp_gu.resize((size_t)c.n_experts); L.exp_down.resize((size_t)c.n_experts); L.exp_have.assign((size_t)c.n_experts, 0); }
  *out = m;
  return CAI_OK;
}

// Expert-parallel twin of cai_model_create for mixture-of-experts models: the dense parts (attention, router,
// embeddings) are replicated on every rank, rank r keeps experts [r E / n, (r + 1) E / n), and a session holds the
// rank's own sequences (data parallel outside the expert layers). Per expert layer the ranks all-gather their
// tokens' normalised activations with the routing decisions, run the pairs routed to their experts, combine them
// per token and reduce-scatter the partial sums back to the tokens' owners.
int cai_model_create_ep(cai_ctx* ctx, const cai_llama_config* cfg, int ep_rank, int ep_size, cai_model** out) {
  CAI_TRY(cai_bind(ctx));
  if (!cfg || !out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_create_ep: null argument");
  if (ep_size < 1 || ep_rank < 0 || ep_rank >= ep_size) return cai_fail(ctx, CAI_ERR_INVALID, "ep rank %d of %d", ep_rank, ep_size);
  if (ep_size > 1) {
    if (cfg->n_experts < 1 || (cfg->n_experts % ep_size)) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "expert parallelism needs n_experts divisible by ep_size");
    if (comm_world(ctx) != ep_size || comm_rank(ctx) != ep_rank) return cai_fail(ctx, CAI_ERR_STATE, "call cai_comm_init with this rank and world == ep_size first");
  }
  CAI_TRY(cai_model_create(ctx, cfg, 0, 1, out));
  (*out)->ep_rank = ep_rank;
  (*out)->ep_size = ep_size;
  return CAI_OK;
}

int cai_model_destroy(cai_model* m) {
  if (!m) return CAI_ERR_INVALID;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  for (auto& L : m->layers) layer_free(L);
  qweight_free(&m->embed);
  qweight_free(&m->lm_head);
  if (m->final_norm) cudaFree(m->final_norm);
  if (m->theta) cudaFree(m->theta);
  delete m;
  return CAI_OK;
}

int cai_model_upload_tensor(cai_model* m, const char* hf_name, int type, const void* data_host, int64_t rows, int64_t cols,
                            int interleave_head_dim) {
  if (!m) return CAI_ERR_INVALID;
  cai_ctx* ctx = m->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!hf_name || !data_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_upload_tensor: null argument");
  if (m->sessions > 0) return cai_fail(ctx, CAI_ERR_STATE, "weights are immutable while sessions exist");
  const cai_llama_config& c = m->cfg;
  const TName t = parse_name(hf_name);
  {
    // Formats no kernel reads directly are decoded to fp32 here and continue as F32 tensors. The resident K-quants
    // take the same route when the int8 switch is on (int8 rows are made from fp32 rows) and when a tensor-parallel
    // column split of O / down would cut through a 256-element super-block.
    bool decode = gguf_type_needs_decode(type);
    if (cai_type_is_kquant(type)) {
      if (m->int8_weights) decode = true;
      if (m->tp_size > 1 && ((t.kind == T_O && (m->qw_l % 256)) || (t.kind == T_DOWN && (m->inter_l % 256)))) decode = true;
      if (rows == 1 || t.kind == T_ROUTER) decode = true;         // vectors are fp32 on the device; the router stays on the plain path
    }
    if (decode) return gguf_upload_decoded(m, ctx, hf_name, type, data_host, rows, cols, interleave_head_dim);
  }
  if (t.kind == T_IGNORE) return CAI_OK;
  if (t.kind == T_UNKNOWN) return cai_fail(ctx, CAI_ERR_INVALID, "unknown tensor name '%s'", hf_name);
  if (t.layer >= c.layers) return cai_fail(ctx, CAI_ERR_INVALID, "'%s': layer %d of %d", hf_name, t.layer, c.layers);
  const int H = c.hidden, QW = c.heads * c.head_dim, KW = c.kv_heads * c.head_dim;
  const int r = m->tp_rank;
  auto shape_is = [&](int64_t er, int64_t ec) -> bool { return rows == er && cols == ec; };
  auto vec_len = [&]() -> int64_t { return rows * cols; };
#define NEED_SHAPE(er, ec)                                                                                      \
  if (!shape_is((er), (ec)))                                                                                    \
    return cai_fail(ctx, CAI_ERR_INVALID, "'%s': shape %lld x %lld, expected %lld x %lld", hf_name,              \
                    (long long)rows, (long long)cols, (long long)(er), (long long)(ec))
#define NEED_VEC(n)                                                                                             \
  if (type != CAI_TYPE_F32 || vec_len() != (n))                                                                 \
    return cai_fail(ctx, CAI_ERR_INVALID, "'%s': expected an F32 vector of %lld", hf_name, (long long)(n))
  m->finalized = false;
  // the importer's pQuantizeInt8: F32 matrices become int8 rows (one fp32 scale per row) as they arrive
  const bool q8 = m->int8_weights && type == CAI_TYPE_F32;
  const int stype = q8 ? CAI_TYPE_I8ROW : type;
  auto put = [&](QWeight* w, int64_t row0, int64_t col0, int interleave) -> int {
    if (q8) return qweight_upload_quantize_i8(ctx, w, (const float*)data_host, rows, cols, row0, col0, interleave);
    return qweight_upload(ctx, w, data_host, rows, cols, row0, col0, interleave);
  };
  switch (t.kind) {
    case T_EMBED: {
      NEED_SHAPE(c.vocab, H);
      CAI_TRY(ensure_weight(ctx, &m->embed, stype, c.vocab, H));
      CAI_TRY(put(&m->embed, 0, 0, 0));
      m->have_embed = true;
      return CAI_OK;
    }
    case T_LM_HEAD: {
      NEED_SHAPE(c.vocab, H);
      CAI_TRY(ensure_weight(ctx, &m->lm_head, stype, m->vocab_l, H));
      CAI_TRY(put(&m->lm_head, (int64_t)r * m->vocab_l, 0, 0));
      m->have_head = true;
      return CAI_OK;
    }
    case T_FINAL_NORM: {
      NEED_VEC(H);
      CAI_TRY(ensure_vec(ctx, &m->final_norm, H, false));
      return upload_vec(ctx, m->final_norm, (const float*)data_host, H, 0, H, 0);
    }
    default: break;
  }
  LayerW& L = m->layers[(size_t)t.layer];
  const int qkv_rows = m->qw_l + 2 * m->kw_l;
  switch (t.kind) {
    case T_ATTN_NORM: NEED_VEC(H); CAI_TRY(ensure_vec(ctx, &L.attn_norm, H, false)); L.have |= HAVE_ATTN_NORM;
      return upload_vec(ctx, L.attn_norm, (const float*)data_host, H, 0, H, 0);
    case T_FFN_NORM: NEED_VEC(H); CAI_TRY(ensure_vec(ctx, &L.ffn_norm, H, false)); L.have |= HAVE_FFN_NORM;
      return upload_vec(ctx, L.ffn_norm, (const float*)data_host, H, 0, H, 0);
    case T_QNORM: NEED_VEC(QW); CAI_TRY(ensure_vec(ctx, &L.q_norm, QW, false)); L.have |= HAVE_QNORM;
      return upload_vec(ctx, L.q_norm, (const float*)data_host, QW, 0, QW, interleave_head_dim);
    case T_KNORM: NEED_VEC(KW); CAI_TRY(ensure_vec(ctx, &L.k_norm, KW, false)); L.have |= HAVE_KNORM;
      return upload_vec(ctx, L.k_norm, (const float*)data_host, KW, 0, KW, interleave_head_dim);
    case T_Q: case T_K: case T_V: {
      const bool isq = t.kind == T_Q;
      NEED_SHAPE(isq ? QW : KW, H);
      const int64_t nloc = isq ? m->qw_l : m->kw_l;
      const int64_t dst0 = isq ? 0 : (t.kind == T_K ? m->qw_l : m->qw_l + m->kw_l);
      const int part = isq ? 0 : (t.kind == T_K ? 1 : 2);
      if (!L.qkv_split && L.wqkv.codes && L.wqkv.type != stype) {
        // a member in another format than the ones before it: the group continues as separate matrices
        const int64_t row0[3] = {0, m->qw_l, m->qw_l + m->kw_l}, nrows[3] = {m->qw_l, m->kw_l, m->kw_l};
        const bool have[3] = {(L.have & HAVE_Q) != 0, (L.have & HAVE_K) != 0, (L.have & HAVE_V) != 0};
        CAI_TRY(split_fused(ctx, &L.wqkv, L.wq_part, row0, nrows, have, 3));
        L.qkv_split = true;
      }
      if (L.qkv_split) {
        if (L.wq_part[part].codes && L.wq_part[part].type != stype) { L.wq_part[part].bias = nullptr; qweight_free(&L.wq_part[part]); }
        CAI_TRY(ensure_weight(ctx, &L.wq_part[part], stype, nloc, H));
        CAI_TRY(put(&L.wq_part[part], (int64_t)r * nloc, 0, t.kind == T_V ? 0 : interleave_head_dim));
      } else {
        CAI_TRY(ensure_weight(ctx, &L.wqkv, stype, qkv_rows, H));
        QWeight view = qweight_rows_view(L.wqkv, dst0, nloc);
        CAI_TRY(put(&view, (int64_t)r * nloc, 0, t.kind == T_V ? 0 : interleave_head_dim));
      }
      L.have |= isq ? HAVE_Q : (t.kind == T_K ? HAVE_K : HAVE_V);
      return CAI_OK;
    }
    case T_QB: case T_KB: case T_VB: {
      const bool isq = t.kind == T_QB;
      NEED_VEC(isq ? QW : KW);
      CAI_TRY(ensure_vec(ctx, &L.qkv_bias, qkv_rows, true));
      const int64_t nloc = isq ? m->qw_l : m->kw_l;
      const int64_t dst0 = isq ? 0 : (t.kind == T_KB ? m->qw_l : m->qw_l + m->kw_l);
      L.have |= isq ? HAVE_QB : (t.kind == T_KB ? HAVE_KB : HAVE_VB);
      return upload_vec(ctx, L.qkv_bias + dst0, (const float*)data_host, isq ? QW : KW, (int64_t)r * nloc, nloc,
                        t.kind == T_VB ? 0 : interleave_head_dim);
    }
    case T_O: {
      NEED_SHAPE(H, QW);
      CAI_TRY(ensure_weight(ctx, &L.wo, stype, H, m->qw_l));
      CAI_TRY(put(&L.wo, 0, (int64_t)r * m->qw_l, 0));
      L.have |= HAVE_O;
      return CAI_OK;
    }
    case T_GATE: case T_UP: {
      if (c.n_experts) return cai_fail(ctx, CAI_ERR_INVALID, "'%s': dense MLP tensor in an MoE configuration", hf_name);
      NEED_SHAPE(c.inter, H);
      const int part = (t.kind == T_UP) ? 0 : 1;
      if (!L.gu_split && L.wgu.codes && L.wgu.type != stype) {
        const int64_t row0[2] = {0, m->inter_l}, nrows[2] = {m->inter_l, m->inter_l};
        const bool have[2] = {(L.have & HAVE_UP) != 0, (L.have & HAVE_GATE) != 0};
        CAI_TRY(split_fused(ctx, &L.wgu, L.wgu_part, row0, nrows, have, 2));
        L.gu_split = true;
      }
      if (L.gu_split) {
        if (L.wgu_part[part].codes && L.wgu_part[part].type != stype) qweight_free(&L.wgu_part[part]);
        CAI_TRY(ensure_weight(ctx, &L.wgu_part[part], stype, m->inter_l, H));
        CAI_TRY(put(&L.wgu_part[part], (int64_t)r * m->inter_l, 0, 0));
      } else {
        CAI_TRY(ensure_weight(ctx, &L.wgu, stype, 2 * (int64_t)m->inter_l, H));
        // up rows first, gate rows second
        QWeight view = qweight_rows_view(L.wgu, part == 0 ? 0 : m->inter_l, m->inter_l);
        CAI_TRY(put(&view, (int64_t)r * m->inter_l, 0, 0));
      }
      L.have |= (t.kind == T_UP) ? HAVE_UP : HAVE_GATE;
      return CAI_OK;
    }
    case T_DOWN: {
      if (c.n_experts) return cai_fail(ctx, CAI_ERR_INVALID, "'%s': dense MLP tensor in an MoE configuration", hf_name);
      NEED_SHAPE(H, c.inter);
      CAI_TRY(ensure_weight(ctx, &L.wdown, stype, H, m->inter_l));
      CAI_TRY(put(&L.wdown, 0, (int64_t)r * m->inter_l, 0));
      L.have |= HAVE_DOWN;
      return CAI_OK;
    }
    case T_ROUTER: {
      if (!c.n_experts) return cai_fail(ctx, CAI_ERR_INVALID, "'%s': router in a dense configuration", hf_name);
      NEED_SHAPE(c.n_experts, H);
      CAI_TRY(ensure_weight(ctx, &L.router, type, c.n_experts, H));
      CAI_TRY(qweight_upload(ctx, &L.router, data_host, rows, cols, 0, 0, 0));
      L.have |= HAVE_ROUTER;
      return CAI_OK;
    }
    case T_EXP_GATE: case T_EXP_UP: case T_EXP_DOWN: {
      if (!c.n_experts || t.expert < 0 || t.expert >= c.n_experts) return cai_fail(ctx, CAI_ERR_INVALID, "'%s': expert index", hf_name);
      if (!m->owns_expert(t.expert)) return CAI_OK;         // expert parallelism: another rank keeps this expert
      const int Im = c.moe_inter;
      if (t.kind == T_EXP_DOWN) {
        NEED_SHAPE(H, Im);
        QWeight* w = &L.exp_down[(size_t)t.expert];
        CAI_TRY(ensure_weight(ctx, w, type, H, Im));
        CAI_TRY(qweight_upload(ctx, w, data_host, rows, cols, 0, 0, 0));
        L.exp_have[(size_t)t.expert] |= 4;
      } else {
        NEED_SHAPE(Im, H);
        QWeight* w = &L.exp_gu[(size_t)t.expert];
        CAI_TRY(ensure_weight(ctx, w, type, 2 * (int64_t)Im, H));
        QWeight view = qweight_rows_view(*w, t.kind == T_EXP_UP ? 0 : Im, Im);
        CAI_TRY(qweight_upload(ctx, &view, data_host, rows, cols, 0, 0, 0));
        w->present = true;
        L.exp_have[(size_t)t.expert] |= (t.kind == T_EXP_UP) ? 2 : 1;
      }
      return CAI_OK;
    }
    default: break;
  }
#undef NEED_SHAPE
#undef NEED_VEC
  return cai_fail(ctx, CAI_ERR_INVALID, "'%s': unhandled tensor", hf_name);
}

int cai_model_set_int8_weights(cai_model* m, int on) {
  if (!m) return CAI_ERR_INVALID;
  cai_ctx* ctx = m->ctx;
  if (m->sessions > 0) return cai_fail(ctx, CAI_ERR_STATE, "weights are immutable while sessions exist");
  if (on && (m->cfg.n_experts > 0 || m->tp_size > 1))
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "int8-on-upload covers dense single-GPU models (a row's scale spans the whole row; expert banks keep their storage type)");
  m->int8_weights = on != 0;
  return CAI_OK;
}

int cai_model_init_synthetic(cai_model* m, int type, uint64_t seed, float std) {
  if (!m) return CAI_ERR_INVALID;
  cai_ctx* ctx = m->ctx;
  CAI_TRY(cai_bind(ctx));
  if (m->sessions > 0) return cai_fail(ctx, CAI_ERR_STATE, "weights are immutable while sessions exist");
  const cai_llama_config& c = m->cfg;
  const int H = c.hidden, QW = c.heads * c.head_dim, KW = c.kv_heads * c.head_dim, r = m->tp_rank;
  if ((H % 32) || (QW % 32) || (c.n_experts ? (c.moe_inter % 32) : (c.inter % 32)))
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "synthetic init needs 32-aligned widths");
  if (type == CAI_TYPE_I8ROW && (c.n_experts > 0 || m->tp_size > 1))
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "synthetic int8 rows cover dense single-GPU models");
  m->finalized = false;
  CAI_TRY(ensure_weight(ctx, &m->embed, type, c.vocab, H));
  CAI_TRY(qweight_init_synthetic(ctx, &m->embed, seed, 9000, std, 0, 0, H));
  m->have_embed = true;
  if (!c.tie_embeddings) {
    CAI_TRY(ensure_weight(ctx, &m->lm_head, type, m->vocab_l, H));
    CAI_TRY(qweight_init_synthetic(ctx, &m->lm_head, seed, 9001, std, (int64_t)r * m->vocab_l, 0, H));
    m->have_head = true;
  }
  CAI_TRY(ensure_vec(ctx, &m->final_norm, H, false));
  CAI_TRY(vec_init_synthetic(ctx, m->final_norm, H, seed, 0, 0.f, 0, 1.0f));
  for (int l = 0; l < c.layers; ++l) {
    LayerW& L = m->layers[(size_t)l];
    const uint64_t tid = 100 + (uint64_t)l * 32;
    CAI_TRY(ensure_vec(ctx, &L.attn_norm, H, false));
    CAI_TRY(vec_init_synthetic(ctx, L.attn_norm, H, seed, 0, 0.f, 0, 1.0f));
    CAI_TRY(ensure_vec(ctx, &L.ffn_norm, H, false));
    CAI_TRY(vec_init_synthetic(ctx, L.ffn_norm, H, seed, 0, 0.f, 0, 1.0f));
    L.have |= HAVE_ATTN_NORM | HAVE_FFN_NORM;
    CAI_TRY(ensure_weight(ctx, &L.wqkv, type, m->qw_l + 2 * m->kw_l, H));
    {
      QWeight vq = qweight_rows_view(L.wqkv, 0, m->qw_l);
      QWeight vk = qweight_rows_view(L.wqkv, m->qw_l, m->kw_l);
      QWeight vv = qweight_rows_view(L.wqkv, m->qw_l + m->kw_l, m->kw_l);
      CAI_TRY(qweight_init_synthetic(ctx, &vq, seed, tid + 0, std, (int64_t)r * m->qw_l, 0, H));
      CAI_TRY(qweight_init_synthetic(ctx, &vk, seed, tid + 1, std, (int64_t)r * m->kw_l, 0, H));
      CAI_TRY(qweight_init_synthetic(ctx, &vv, seed, tid + 2, std, (int64_t)r * m->kw_l, 0, H));
      L.wqkv.present = true;
      L.have |= HAVE_Q | HAVE_K | HAVE_V;
    }
    if (c.qkv_bias) {
      CAI_TRY(ensure_vec(ctx, &L.qkv_bias, m->qw_l + 2 * m->kw_l, true));
      CAI_TRY(vec_init_synthetic(ctx, L.qkv_bias, m->qw_l, seed, tid + 3, std, (int64_t)r * m->qw_l, 0.f));
      CAI_TRY(vec_init_synthetic(ctx, L.qkv_bias + m->qw_l, m->kw_l, seed, tid + 4, std, (int64_t)r * m->kw_l, 0.f));
      CAI_TRY(vec_init_synthetic(ctx, L.qkv_bias + m->qw_l + m->kw_l, m->kw_l, seed, tid + 5, std, (int64_t)r * m->kw_l, 0.f));
      L.have |= HAVE_QB | HAVE_KB | HAVE_VB;
    }
    if (c.qk_norm) {
      CAI_TRY(ensure_vec(ctx, &L.q_norm, QW, false));
      CAI_TRY(vec_init_synthetic(ctx, L.q_norm, QW, seed, 0, 0.f, 0, 1.0f));
      CAI_TRY(ensure_vec(ctx, &L.k_norm, KW, false));
      CAI_TRY(vec_init_synthetic(ctx, L.k_norm, KW, seed, 0, 0.f, 0, 1.0f));
      L.have |= HAVE_QNORM | HAVE_KNORM;
    }
    CAI_TRY(ensure_weight(ctx, &L.wo, type, H, m->qw_l));
    CAI_TRY(qweight_init_synthetic(ctx, &L.wo, seed, tid + 6, std, 0, (int64_t)r * m->qw_l, QW));
    L.have |= HAVE_O;
    if (!c.n_experts) {
      CAI_TRY(ensure_weight(ctx, &L.wgu, type, 2 * (int64_t)m->inter_l, H));
      QWeight vu = qweight_rows_view(L.wgu, 0, m->inter_l);
      QWeight vg = qweight_rows_view(L.wgu, m->inter_l, m->inter_l);
      CAI_TRY(qweight_init_synthetic(ctx, &vu, seed, tid + 7, std, (int64_t)r * m->inter_l, 0, H));
      CAI_TRY(qweight_init_synthetic(ctx, &vg, seed, tid + 8, std, (int64_t)r * m->inter_l, 0, H));
      L.wgu.present = true;
      CAI_TRY(ensure_weight(ctx, &L.wdown, type, H, m->inter_l));
      CAI_TRY(qweight_init_synthetic(ctx, &L.wdown, seed, tid + 9, std, 0, (int64_t)r * m->inter_l, c.inter));
      L.have |= HAVE_GATE | HAVE_UP | HAVE_DOWN;
    } else {
      const int Im = c.moe_inter;
      CAI_TRY(ensure_weight(ctx, &L.router, type, c.n_experts, H));
      CAI_TRY(qweight_init_synthetic(ctx, &L.router, seed, tid + 10, std, 0, 0, H));
      L.have |= HAVE_ROUTER;
      for (int e = 0; e < c.n_experts; ++e) {
        if (!m->owns_expert(e)) continue;
        const uint64_t etid = 100000 + ((uint64_t)l * (uint64_t)c.n_experts + (uint64_t)e) * 4;
        QWeight* gu = &L.exp_gu[(size_t)e];
        CAI_TRY(ensure_weight(ctx, gu, type, 2 * (int64_t)Im, H));
        QWeight vu = qweight_rows_view(*gu, 0, Im);
        QWeight vg = qweight_rows_view(*gu, Im, Im);
        CAI_TRY(qweight_init_synthetic(ctx, &vu, seed, etid + 0, std, 0, 0, H));
        CAI_TRY(qweight_init_synthetic(ctx, &vg, seed, etid + 1, std, 0, 0, H));
        gu->present = true;
        QWeight* dn = &L.exp_down[(size_t)e];
        CAI_TRY(ensure_weight(ctx, dn, type, H, Im));
        CAI_TRY(qweight_init_synthetic(ctx, dn, seed, etid + 2, std, 0, 0, Im));
        L.exp_have[(size_t)e] = 7;
      }
    }
  }
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

// Resolves a tensor name to the resident storage (view) it was placed in.
static int locate_tensor(cai_model* m, const char* hf_name, QWeight* out_view, const float** out_vec, int64_t* out_vec_len) {
  cai_ctx* ctx = m->ctx;
  const TName t = parse_name(hf_name);
  *out_vec = nullptr; *out_vec_len = 0;
  if (t.kind == T_UNKNOWN || t.kind == T_IGNORE || t.layer >= m->cfg.layers) return cai_fail(ctx, CAI_ERR_INVALID, "unknown tensor name '%s'", hf_name);
  const cai_llama_config& c = m->cfg;
  if (t.kind == T_EMBED) { *out_view = qweight_rows_view(m->embed, 0, m->embed.n); return CAI_OK; }
  if (t.kind == T_LM_HEAD) { *out_view = qweight_rows_view(m->lm_head, 0, m->lm_head.n); return CAI_OK; }
  if (t.kind == T_FINAL_NORM) { *out_vec = m->final_norm; *out_vec_len = c.hidden; return CAI_OK; }
  LayerW& L = m->layers[(size_t)t.layer];
  switch (t.kind) {
    case T_ATTN_NORM: *out_vec = L.attn_norm; *out_vec_len = c.hidden; return CAI_OK;
    case T_FFN_NORM: *out_vec = L.ffn_norm; *out_vec_len = c.hidden; return CAI_OK;
    case T_QNORM: *out_vec = L.q_norm; *out_vec_len = c.heads * c.head_dim; return CAI_OK;
    case T_KNORM: *out_vec = L.k_norm; *out_vec_len = c.kv_heads * c.head_dim; return CAI_OK;
    case T_Q: *out_view = L.qkv_split ? qweight_rows_view(L.wq_part[0], 0, m->qw_l) : qweight_rows_view(L.wqkv, 0, m->qw_l); return CAI_OK;
    case T_K: *out_view = L.qkv_split ? qweight_rows_view(L.wq_part[1], 0, m->kw_l) : qweight_rows_view(L.wqkv, m->qw_l, m->kw_l); return CAI_OK;
    case T_V: *out_view = L.qkv_split ? qweight_rows_view(L.wq_part[2], 0, m->kw_l) : qweight_rows_view(L.wqkv, m->qw_l + m->kw_l, m->kw_l); return CAI_OK;
    case T_QB: *out_vec = L.qkv_bias; *out_vec_len = m->qw_l; return CAI_OK;
    case T_KB: *out_vec = L.qkv_bias ? L.qkv_bias + m->qw_l : nullptr; *out_vec_len = m->kw_l; return CAI_OK;
    case T_VB: *out_vec = L.qkv_bias ? L.qkv_bias + m->qw_l + m->kw_l : nullptr; *out_vec_len = m->kw_l; return CAI_OK;
    case T_O: *out_view = qweight_rows_view(L.wo, 0, L.wo.n); return CAI_OK;
    case T_UP: *out_view = L.gu_split ? qweight_rows_view(L.wgu_part[0], 0, m->inter_l) : qweight_rows_view(L.wgu, 0, m->inter_l); return CAI_OK;
    case T_GATE: *out_view = L.gu_split ? qweight_rows_view(L.wgu_part[1], 0, m->inter_l) : qweight_rows_view(L.wgu, m->inter_l, m->inter_l); return CAI_OK;
    case T_DOWN: *out_view = qweight_rows_view(L.wdown, 0, L.wdown.n); return CAI_OK;
    case T_ROUTER: *out_view = qweight_rows_view(L.router, 0, L.router.n); return CAI_OK;
    case T_EXP_UP: case T_EXP_GATE: case T_EXP_DOWN: {
      if (t.expert < 0 || t.expert >= c.n_experts) return cai_fail(ctx, CAI_ERR_INVALID, "'%s': expert index", hf_name);
      if (t.kind == T_EXP_DOWN) *out_view = qweight_rows_view(L.exp_down[(size_t)t.expert], 0, c.hidden);
      else *out_view = qweight_rows_view(L.exp_gu[(size_t)t.expert], t.kind == T_EXP_UP ? 0 : c.moe_inter, c.moe_inter);
      return CAI_OK;
    }
    default: break;
  }
  return cai_fail(ctx, CAI_ERR_INVALID, "'%s': unhandled tensor", hf_name);
}

int cai_model_read_tensor(cai_model* m, const char* hf_name, void* out_host, int64_t out_bytes_cap, int* out_type,
                          int64_t* out_rows, int64_t* out_cols) {
  if (!m) return CAI_ERR_INVALID;
  cai_ctx* ctx = m->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!hf_name || !out_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_read_tensor: null argument");
  QWeight view; const float* vec = nullptr; int64_t vlen = 0;
  CAI_TRY(locate_tensor(m, hf_name, &view, &vec, &vlen));
  if (vlen > 0) {
    if (!vec) return cai_fail(ctx, CAI_ERR_STATE, "'%s' has not been uploaded", hf_name);
    if (vlen * 4 > out_bytes_cap) return cai_fail(ctx, CAI_ERR_INVALID, "host buffer too small");
    CAI_CUDA(ctx, cudaMemcpyAsync(out_host, vec, (size_t)vlen * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (out_type) *out_type = CAI_TYPE_F32;
    if (out_rows) *out_rows = 1;
    if (out_cols) *out_cols = vlen;
    return CAI_OK;
  }
  if (!view.codes) return cai_fail(ctx, CAI_ERR_STATE, "'%s' has not been uploaded", hf_name);
  CAI_TRY(qweight_download_blocks(ctx, &view, out_host, (size_t)out_bytes_cap));
  if (out_type) *out_type = view.type;
  if (out_rows) *out_rows = view.n;
  if (out_cols) *out_cols = view.k;
  return CAI_OK;
}

static int upload_ptr_array(cai_ctx* ctx, const void*** dst, const std::vector<const void*>& src) {
  if (*dst) cudaFree((void*)*dst);
  *dst = nullptr;
  CAI_CUDA(ctx, cudaMalloc((void**)dst, src.size() * sizeof(void*)));
  CAI_CUDA(ctx, cudaMemcpyAsync((void*)*dst, src.data(), src.size() * sizeof(void*), cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

int cai_model_finalize(cai_model* m) {
  if (!m) return CAI_ERR_INVALID;
  cai_ctx* ctx = m->ctx;
  CAI_TRY(cai_bind(ctx));
  const cai_llama_config& c = m->cfg;
  if (!m->have_embed) return cai_fail(ctx, CAI_ERR_STATE, "missing tensor model.embed_tokens.weight");
  if (!m->final_norm) return cai_fail(ctx, CAI_ERR_STATE, "missing tensor model.norm.weight");
  if (!m->have_head) {
    // tied head = the embedding rows (this rank's vocabulary shard)
    if (!c.tie_embeddings) return cai_fail(ctx, CAI_ERR_STATE, "missing tensor lm_head.weight (and tie_embeddings is off)");
    m->lm_head = qweight_rows_view(m->embed, (int64_t)m->tp_rank * m->vocab_l, m->vocab_l);
    m->have_head = true;
  }
  for (int l = 0; l < c.layers; ++l) {
    LayerW& L = m->layers[(size_t)l];
    uint32_t need = HAVE_ATTN_NORM | HAVE_FFN_NORM | HAVE_Q | HAVE_K | HAVE_V | HAVE_O;
    if (c.qkv_bias) need |= HAVE_QB | HAVE_KB | HAVE_VB;
    if (c.qk_norm) need |= HAVE_QNORM | HAVE_KNORM;
    if (c.n_experts) need |= HAVE_ROUTER; else need |= HAVE_GATE | HAVE_UP | HAVE_DOWN;
    if ((L.have & need) != need) return cai_fail(ctx, CAI_ERR_STATE, "layer %d is missing tensors (have mask 0x%x, need 0x%x)", l, L.have, need);
    L.wqkv.bias = L.qkv_bias;     // alias; freed through qkv_bias
    if (L.qkv_split && L.qkv_bias) {
      L.wq_part[0].bias = L.qkv_bias; L.wq_part[1].bias = L.qkv_bias + m->qw_l; L.wq_part[2].bias = L.qkv_bias + m->qw_l + m->kw_l;
    }
    if (c.n_experts) {
      std::vector<const void*> gc, gs, dc, ds;
      const int e0 = m->expert_lo();
      for (int e = 0; e < c.n_experts; ++e) {
        if (!m->owns_expert(e)) { gc.push_back(nullptr); gs.push_back(nullptr); dc.push_back(nullptr); ds.push_back(nullptr); continue; }
        if (L.exp_have[(size_t)e] != 7) return cai_fail(ctx, CAI_ERR_STATE, "layer %d expert %d is missing tensors", l, e);
        if (L.exp_gu[(size_t)e].type != L.exp_gu[(size_t)e0].type || L.exp_down[(size_t)e].type != L.exp_down[(size_t)e0].type)
          return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "experts of one layer must share a storage type");
        gc.push_back(L.exp_gu[(size_t)e].codes); gs.push_back(L.exp_gu[(size_t)e].scales);
        dc.push_back(L.exp_down[(size_t)e].codes); ds.push_back(L.exp_down[(size_t)e].scales);
      }
      CAI_TRY(upload_ptr_array(ctx, &L.d_gu_codes, gc));
      CAI_TRY(upload_ptr_array(ctx, (const void***)&L.d_gu_scales, gs));
      CAI_TRY(upload_ptr_array(ctx, &L.d_down_codes, dc));
      CAI_TRY(upload_ptr_array(ctx, (const void***)&L.d_down_scales, ds));
    }
  }
  if (!m->theta) CAI_CUDA(ctx, cudaMalloc((void**)&m->theta, (size_t)(c.head_dim / 2) * 4));
  CAI_TRY(op_rope_theta_table(ctx, m->theta, c.head_dim, c.rope_theta));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  m->finalized = true;
  return CAI_OK;
}

int cai_model_step_weight_bytes(cai_model* m, int64_t* out_bytes) {
  if (!m || !out_bytes) return CAI_ERR_INVALID;
  if (!m->finalized) return cai_fail(m->ctx, CAI_ERR_STATE, "model is not finalized");
  int64_t b = (int64_t)m->lm_head.bytes();
  for (auto& L : m->layers) {
    b += (int64_t)(L.wqkv.bytes() + L.wo.bytes());
    if (L.qkv_split) for (const QWeight& w : L.wq_part) b += (int64_t)w.bytes();
    if (L.gu_split) for (const QWeight& w : L.wgu_part) b += (int64_t)w.bytes();
    if (m->cfg.n_experts) {
      b += (int64_t)L.router.bytes();
      // one token touches top_k experts
      b += (int64_t)m->cfg.top_k * (int64_t)(L.exp_gu[(size_t)m->expert_lo()].bytes() + L.exp_down[(size_t)m->expert_lo()].bytes());
    } else {
      b += (int64_t)(L.wgu.bytes() + L.wdown.bytes());
    }
  }
  *out_bytes = b;
  return CAI_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// session
// ---------------------------------------------------------------------------
struct cai_session {
  cai_model* m;
  cai_ctx* ctx;
  int max_ctx, batch;
  int ctx_pitch = 0;                                  // positions per KV head in the caches: max_ctx rounded up to 32
  int k_blocked = 0;                                  // K cache block-transposed (cai_k_blocked_index)
  int window = 0;                                     // > 0: every layer attends over the most recent `window` rows only
  int evict_sinks = 0, evict_window = 0;              // evict_window > 0: StreamingLLM (sinks + a ring of recent rows)
  float *k_cache = nullptr, *v_cache = nullptr;       // [layers][B][kv_heads_l][ctx_pitch][hd]; int8 codes when kv_int8
  float *k_snap = nullptr, *v_snap = nullptr;
  size_t layer_stride = 0;                            // elements per layer
  // chunked prefill: a helper session of C rows per sequence that BORROWS this session's caches (kv_owner set in the
  // helper: its rows are consecutive positions of the owner's sequences, seq_index_dev says which) and stops before
  // the LM head
  cai_session* wide = nullptr;
  cai_session* kv_owner = nullptr;
  int32_t* seq_index_dev = nullptr;
  int wide_chunk = 0;                                 // positions per sequence and helper step
  bool kv_int8 = false;                               // the reference's int8 cache: codes above + one fp32 scale per row
  float *k_scales = nullptr, *v_scales = nullptr;     // [layers][B][kv_heads_l][max_ctx]
  float *k_scales_snap = nullptr, *v_scales_snap = nullptr;
  size_t scale_stride = 0;                            // scales per layer
  size_t cache_bytes() const { return layer_stride * (size_t)m->cfg.layers * (kv_int8 ? 1 : 4); }
  size_t scale_bytes() const { return scale_stride * (size_t)m->cfg.layers * 4; }
  int32_t *tokens_dev = nullptr, *pos_dev = nullptr, *len_dev = nullptr;
  int32_t* io_pinned = nullptr;                       // [4][B] tokens, pos, len, sequence index
  std::vector<int32_t> len_host, len_snap;
  bool have_snap = false;
  float *x = nullptr, *x_alt = nullptr, *h = nullptr, *qkv = nullptr, *att = nullptr, *act = nullptr, *logits = nullptr;
  float* gu = nullptr;                                // [B][2*inter] un-fused up|gate (tensor-core batches)
  float *router_logits = nullptr, *gates = nullptr, *moe_hidden = nullptr, *pair_out = nullptr;
  int32_t* expert_ids = nullptr;
  // grouped (tensor-core) expert path: pairs sorted into 16-row tiles per expert
  int moe_tiles = 0;                       // 0 = the per-pair GEMV path
  int32_t *tile_expert = nullptr, *tile_pairs = nullptr;
  float *moe_gu = nullptr, *moe_unscale = nullptr;
  void* moe_xp = nullptr;
  // expert parallelism: the gathered tokens of all ranks
  float *ep_pack = nullptr, *ep_all = nullptr, *ep_gates = nullptr, *ep_part = nullptr, *ep_mine = nullptr;
  int32_t* ep_ids = nullptr;
  float* partial = nullptr;
  int nsplit = 1;
  int32_t* amax_idx = nullptr; float* amax_val = nullptr;
  float* amax_part_val = nullptr; int* amax_part_idx = nullptr; int* amax_tickets = nullptr;
  float* rope_cs = nullptr;                           // [B][head_dim/2][2] cos/sin of the current step
  float *amax_pack = nullptr, *amax_gather = nullptr, *logits_gather = nullptr;
  int32_t* trace = nullptr; int32_t* trace_count = nullptr; int64_t trace_cap = 0;
  int32_t* prefill_buf = nullptr; int64_t prefill_cap = 0;
  cai_tp_ar* ar = nullptr;                            // peer-memory all-reduce (tensor parallel), NULL = NCCL
  cudaGraphExec_t graph_exec = nullptr;
  int64_t graph_kernels = 0;
  bool use_graph = true;
  int use_pdl = 0;            // programmatic dependent launch for this session's step kernels
  std::vector<float> host_gather;
  // one persistent kernel per step (dense, one sequence, Q8_0, fp32 cache); NULL = one launch per operator
  StepPlan* plan = nullptr;
  unsigned long long* plan_ts = nullptr;              // device buffer of the phase trace (cai_session_profile)
  // device sampling (cai_session_step_topk / cai_session_decode_sampled): allocated on first use
  float* sample_scratch = nullptr; int32_t* sample_ids = nullptr; float* sample_probs = nullptr; float* sample_u = nullptr;
};

__global__ void pack_argmax_kernel(const int32_t* idx, const float* val, int batch, int offset, float* pack) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch) { pack[2 * b] = val[b]; pack[2 * b + 1] = __int_as_float(idx[b] + offset); }
}
__global__ void pick_argmax_kernel(const float* gathered, int batch, int world, int32_t* idx) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  float best = -INFINITY; int besti = 0x7fffffff;
  for (int r = 0; r < world; ++r) {
    const float v = gathered[((size_t)r * batch + b) * 2];
    const int i = __float_as_int(gathered[((size_t)r * batch + b) * 2 + 1]);
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
  idx[b] = (besti == 0x7fffffff) ? 0 : besti;
}
// end of step: next token = argmax, position and cache length advance, argmax appended to the trace
__global__ void advance_kernel(int32_t* tokens, int32_t* pos, int32_t* len, const int32_t* amax, int batch,
                               int32_t* trace, int32_t* trace_count, int64_t trace_cap) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const int cnt = *trace_count;
  if (b < batch) {
    tokens[b] = amax[b];
    pos[b] += 1;
    len[b] += 1;
    if ((int64_t)(cnt + 1) * batch <= trace_cap) trace[(int64_t)cnt * batch + b] = amax[b];
  }
  __syncthreads();
  if (b == 0) *trace_count = cnt + 1;
}

static int enqueue_step(cai_session* s) {
  s->ctx->use_pdl = s->use_pdl;
  cai_model* m = s->m;
  cai_ctx* ctx = s->ctx;
  if (s->plan) return step_plan_enqueue(ctx, s->plan, nullptr);
  const cai_llama_config& c = m->cfg;
  const int B = s->batch, H = c.hidden;
  const int QKVW = m->qw_l + 2 * m->kw_l;
  float* x = s->x;
  float* xalt = s->x_alt;
  auto set_rope = [&](LinearArgs& a, int l) {
    a.epilogue = EPI_QKV_ROPE; a.rope_cs = s->rope_cs; a.rope_q_width = m->qw_l; a.rope_kv_width = m->kw_l;
    a.rope_head_dim = c.head_dim; a.rope_kv_heads = m->kv_heads_l; a.rope_max_ctx = s->ctx_pitch; a.k_blocked = s->k_blocked;
    a.k_cache = s->k_cache + (size_t)l * s->layer_stride; a.v_cache = s->v_cache + (size_t)l * s->layer_stride;
    a.cache_len_dev = s->len_dev;
  };
  CAI_TRY(op_embed(ctx, &m->embed, s->tokens_dev, B, x, H));
  CAI_TRY(op_rope_table(ctx, m->theta, s->pos_dev, B, c.head_dim / 2, s->rope_cs));
  // Batches the dispatcher sends to the tensor-core GEMM (9..64 rows; 3..8 on large matrices) get plain epilogues
  // only: RoPE/append and SwiGLU then run as their own kernels.
  const bool tc_batch = linear_uses_tensor_cores(&m->layers[0].wgu, B) || linear_uses_tensor_cores(&m->layers[0].wqkv, B);
  // RoPE + KV append ride in the [q|k|v] epilogue unless q/k need a full-width norm first, the batch runs on the
  // tensor cores, or the cache is int8 (a row's scale needs the whole row)
  const bool fuse_rope = !c.qk_norm && !tc_batch && !s->kv_int8 && !s->kv_owner && !s->evict_window;
  for (int l = 0; l < c.layers; ++l) {
    LayerW& L = m->layers[(size_t)l];
    const bool fuse_rope_l = fuse_rope && !L.qkv_split;
    if (L.qkv_split) {
      // q, k and v in formats of their own: one product each into the [q | k | v] row, plain epilogue
      CAI_TRY(op_rmsnorm(ctx, x, H, L.attn_norm, s->h, H, B, H, c.rms_eps));
      const int64_t off[3] = {0, m->qw_l, m->qw_l + m->kw_l};
      for (int i = 0; i < 3; ++i) {
        LinearArgs a; a.w = &L.wq_part[i]; a.x = s->h; a.ldx = H; a.y = s->qkv + off[i]; a.ldy = QKVW; a.batch = B;
        CAI_TRY(linear_launch(ctx, a));
      }
    } else if (linear_can_fuse_norm(&L.wqkv, B)) {
      LinearArgs a; a.w = &L.wqkv; a.x = x; a.ldx = H; a.y = s->qkv; a.ldy = QKVW; a.batch = B;
      a.norm_gain = L.attn_norm; a.norm_eps = c.rms_eps;
      if (fuse_rope_l) set_rope(a, l);
      CAI_TRY(linear_launch(ctx, a));
    } else {
      CAI_TRY(op_rmsnorm(ctx, x, H, L.attn_norm, s->h, H, B, H, c.rms_eps));
      LinearArgs a; a.w = &L.wqkv; a.x = s->h; a.ldx = H; a.y = s->qkv; a.ldy = QKVW; a.batch = B;
      if (fuse_rope_l) set_rope(a, l);
      CAI_TRY(linear_launch(ctx, a));
    }
    {
      AttnArgs a;
      a.qkv = s->qkv; a.ld = QKVW;
      if (s->kv_int8) {
        a.k_codes = (int8_t*)s->k_cache + (size_t)l * s->layer_stride; a.v_codes = (int8_t*)s->v_cache + (size_t)l * s->layer_stride;
        a.k_scales = s->k_scales + (size_t)l * s->scale_stride; a.v_scales = s->v_scales + (size_t)l * s->scale_stride;
      } else {
        a.k_cache = s->k_cache + (size_t)l * s->layer_stride; a.v_cache = s->v_cache + (size_t)l * s->layer_stride;
      }
      a.seq_index_dev = s->seq_index_dev;
      a.cache_len_dev = s->len_dev; a.batch = B; a.q_heads = m->heads_l; a.kv_heads = m->kv_heads_l;
      a.head_dim = c.head_dim; a.max_ctx = s->ctx_pitch; a.k_blocked = s->k_blocked; a.theta = m->theta; a.pos_dev = s->pos_dev;
      { cai_session* o = s->kv_owner ? s->kv_owner : s; a.window = o->window; a.evict_sinks = o->evict_sinks; a.evict_window = o->evict_window; }
      a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.eps = c.rms_eps;
      a.out = s->att; a.ldo = m->qw_l; a.partial = s->partial; a.nsplit = s->nsplit;
      if (!fuse_rope_l) CAI_TRY(attn_rope_append(ctx, a));
      CAI_TRY(attn_decode(ctx, a));
    }
    // attention output projection + residual
    if (m->tp_size == 1) {
      LinearArgs a; a.w = &L.wo; a.x = s->att; a.ldx = m->qw_l; a.y = x; a.ldy = H; a.batch = B; a.epilogue = EPI_RESID; a.resid = x;
      CAI_TRY(linear_launch(ctx, a));
    } else if (s->ar) {
      // partial result straight into the peer-visible slot, then one kernel: x_new = x + sum over ranks
      LinearArgs a; a.w = &L.wo; a.x = s->att; a.ldx = m->qw_l; a.y = comm_ar_slot(s->ar, 2 * l); a.ldy = H; a.batch = B;
      CAI_TRY(linear_launch(ctx, a));
      CAI_TRY(comm_ar_reduce(ctx, s->ar, 2 * l, (int64_t)B * H, x, xalt));
      float* t = x; x = xalt; xalt = t;
    } else {
      LinearArgs a; a.w = &L.wo; a.x = s->att; a.ldx = m->qw_l; a.y = xalt; a.ldy = H; a.batch = B;
      if (m->tp_rank == 0) { a.epilogue = EPI_RESID; a.resid = x; }
      CAI_TRY(linear_launch(ctx, a));
      CAI_TRY(comm_allreduce(ctx, xalt, (int64_t)B * H));
      float* t = x; x = xalt; xalt = t;
    }
    const bool fuse_ffn_norm = !c.n_experts && !L.gu_split && linear_can_fuse_norm(&L.wgu, B);
    if (!fuse_ffn_norm) CAI_TRY(op_rmsnorm(ctx, x, H, L.ffn_norm, s->h, H, B, H, c.rms_eps));
    if (!c.n_experts) {
      {
        if (L.gu_split) {
          // up and gate in formats of their own: one product each into the [up | gate] row, then the gated activation
          const int64_t I2 = 2 * (int64_t)m->inter_l;
          for (int i = 0; i < 2; ++i) {
            LinearArgs a; a.w = &L.wgu_part[i]; a.x = s->h; a.ldx = H; a.y = s->gu + (int64_t)i * m->inter_l; a.ldy = I2; a.batch = B;
            CAI_TRY(linear_launch(ctx, a));
          }
          CAI_TRY(op_swiglu(ctx, s->gu, I2, s->act, m->inter_l, B, m->inter_l));
        } else if (tc_batch && s->gu) {
          LinearArgs a; a.w = &L.wgu; a.x = fuse_ffn_norm ? x : s->h; a.ldx = H; a.y = s->gu; a.ldy = 2 * (int64_t)m->inter_l; a.batch = B;
          if (fuse_ffn_norm) { a.norm_gain = L.ffn_norm; a.norm_eps = c.rms_eps; }
          CAI_TRY(linear_launch(ctx, a));
          CAI_TRY(op_swiglu(ctx, s->gu, 2 * (int64_t)m->inter_l, s->act, m->inter_l, B, m->inter_l));
        } else {
          LinearArgs a; a.w = &L.wgu; a.x = fuse_ffn_norm ? x : s->h; a.ldx = H; a.y = s->act; a.ldy = m->inter_l; a.batch = B; a.epilogue = EPI_SWIGLU;
          if (fuse_ffn_norm) { a.norm_gain = L.ffn_norm; a.norm_eps = c.rms_eps; }
          CAI_TRY(linear_launch(ctx, a));
        }
      }
      if (m->tp_size == 1) {
        LinearArgs a; a.w = &L.wdown; a.x = s->act; a.ldx = m->inter_l; a.y = x; a.ldy = H; a.batch = B; a.epilogue = EPI_RESID; a.resid = x;
        CAI_TRY(linear_launch(ctx, a));
      } else if (s->ar) {
        LinearArgs a; a.w = &L.wdown; a.x = s->act; a.ldx = m->inter_l; a.y = comm_ar_slot(s->ar, 2 * l + 1); a.ldy = H; a.batch = B;
        CAI_TRY(linear_launch(ctx, a));
        CAI_TRY(comm_ar_reduce(ctx, s->ar, 2 * l + 1, (int64_t)B * H, x, xalt));
        float* t = x; x = xalt; xalt = t;
      } else {
        LinearArgs a; a.w = &L.wdown; a.x = s->act; a.ldx = m->inter_l; a.y = xalt; a.ldy = H; a.batch = B;
        if (m->tp_rank == 0) { a.epilogue = EPI_RESID; a.resid = x; }
        CAI_TRY(linear_launch(ctx, a));
        CAI_TRY(comm_allreduce(ctx, xalt, (int64_t)B * H));
        float* t = x; x = xalt; xalt = t;
      }
    } else {
      const int E = c.n_experts, K = c.top_k, Im = c.moe_inter;
      {
        LinearArgs a; a.w = &L.router; a.x = s->h; a.ldx = H; a.y = s->router_logits; a.ldy = E; a.batch = B;
        CAI_TRY(linear_launch(ctx, a));
      }
      CAI_TRY(op_topk_gate(ctx, s->router_logits, B, E, K, c.norm_topk, s->expert_ids, s->gates));
      if (m->ep_size > 1) {
        // Expert parallel: gather every rank's rows [h | ids | gates], run the pairs of MY experts for ALL tokens
        // (grouped, on the tensor cores), combine them per token, and reduce-scatter the partial sums to the owners.
        const int Bg = B * m->ep_size, W = (H + 2 * K + 3) & ~3;
        const QWeight& gu = L.exp_gu[(size_t)m->expert_lo()];
        const QWeight& dn = L.exp_down[(size_t)m->expert_lo()];
        if (s->ar) {
          // dispatch over peer memory: rows packed into this rank's slot, then pulled by the ranks that need them
          CAI_TRY(op_moe_pack(ctx, s->h, H, s->expert_ids, s->gates, B, H, K, W, comm_ar_slot(s->ar, 2 * l)));
          CAI_TRY(comm_ep_dispatch(ctx, s->ar, 2 * l, B, W, H, K, m->expert_lo(), m->expert_hi(), s->ep_all, s->ep_ids, s->ep_gates));
        } else {
          CAI_TRY(op_moe_pack(ctx, s->h, H, s->expert_ids, s->gates, B, H, K, W, s->ep_pack));
          CAI_TRY(comm_allgather(ctx, s->ep_pack, s->ep_all, (int64_t)B * W));
          CAI_TRY(op_moe_unpack_ids(ctx, s->ep_all, Bg, H, K, W, s->ep_ids, s->ep_gates));
        }
        CAI_TRY(op_moe_group(ctx, s->ep_ids, Bg * K, E, 16, s->moe_tiles, s->tile_expert, s->tile_pairs, m->expert_lo(), m->expert_hi()));
        ctx->cur_family = FAM_LINEAR;
        CAI_TRY(gemm_tc_launch_grouped(ctx, gu.type, L.d_gu_codes, L.d_gu_scales, gu.n, gu.k, gu.sstride, s->ep_all, W, K, s->moe_gu, 2 * (int64_t)Im,
                                       s->tile_expert, s->tile_pairs, s->moe_tiles, s->moe_xp, s->moe_unscale));
        CAI_TRY(op_swiglu(ctx, s->moe_gu, 2 * (int64_t)Im, s->moe_hidden, Im, Bg * K, Im));
        ctx->cur_family = FAM_LINEAR;
        CAI_TRY(gemm_tc_launch_grouped(ctx, dn.type, L.d_down_codes, L.d_down_scales, dn.n, dn.k, dn.sstride, s->moe_hidden, Im, 1, s->pair_out, H,
                                       s->tile_expert, s->tile_pairs, s->moe_tiles, s->moe_xp, s->moe_unscale));
        if (s->ar) {
          // combine over peer memory: this rank's partial sums of all tokens into its slot; each owner adds what it needs
          CAI_TRY(op_moe_combine_partial(ctx, s->pair_out, H, s->ep_ids, s->ep_gates, Bg, K, H, m->expert_lo(), m->expert_hi(),
                                         comm_ar_slot(s->ar, 2 * l + 1), H));
          CAI_TRY(comm_ep_combine(ctx, s->ar, 2 * l + 1, B, H, K, E / m->ep_size, s->expert_ids, x, H));
        } else {
          CAI_TRY(op_moe_combine_partial(ctx, s->pair_out, H, s->ep_ids, s->ep_gates, Bg, K, H, m->expert_lo(), m->expert_hi(), s->ep_part, H));
          CAI_TRY(comm_reduce_scatter(ctx, s->ep_part, s->ep_mine, (int64_t)B * H));
          CAI_TRY(op_add_rows(ctx, x, H, s->ep_mine, H, B, H));
        }
        continue;
      }
      if (s->moe_tiles) {
        // enough pairs per expert: group them by expert and run each expert's matrices once per 16 pairs on the
        // tensor cores (the per-pair GEMV below streams an expert's weights once per pair)
        const QWeight& gu = L.exp_gu[0];
        const QWeight& dn = L.exp_down[0];
        CAI_TRY(op_moe_group(ctx, s->expert_ids, B * K, E, 16, s->moe_tiles, s->tile_expert, s->tile_pairs, 0, E));
        ctx->cur_family = FAM_LINEAR;
        CAI_TRY(gemm_tc_launch_grouped(ctx, gu.type, L.d_gu_codes, L.d_gu_scales, gu.n, gu.k, gu.sstride, s->h, H, K, s->moe_gu, 2 * (int64_t)Im,
                                       s->tile_expert, s->tile_pairs, s->moe_tiles, s->moe_xp, s->moe_unscale));
        CAI_TRY(op_swiglu(ctx, s->moe_gu, 2 * (int64_t)Im, s->moe_hidden, Im, B * K, Im));
        ctx->cur_family = FAM_LINEAR;
        CAI_TRY(gemm_tc_launch_grouped(ctx, dn.type, L.d_down_codes, L.d_down_scales, dn.n, dn.k, dn.sstride, s->moe_hidden, Im, 1, s->pair_out, H,
                                       s->tile_expert, s->tile_pairs, s->moe_tiles, s->moe_xp, s->moe_unscale));
      } else {
      {
        LinearArgs a; a.w = &L.exp_gu[0]; a.x = s->h; a.ldx = H; a.y = s->moe_hidden; a.ldy = Im; a.batch = B * K;
        a.epilogue = EPI_SWIGLU; a.bank_codes_dev = L.d_gu_codes; a.bank_scales_dev = L.d_gu_scales; a.bank_count = E;
        a.expert_ids_dev = s->expert_ids; a.x_row_div = K;
        CAI_TRY(linear_launch(ctx, a));
      }
      {
        LinearArgs a; a.w = &L.exp_down[0]; a.x = s->moe_hidden; a.ldx = Im; a.y = s->pair_out; a.ldy = H; a.batch = B * K;
        a.bank_codes_dev = L.d_down_codes; a.bank_scales_dev = L.d_down_scales; a.bank_count = E; a.expert_ids_dev = s->expert_ids; a.x_row_div = 1;
        CAI_TRY(linear_launch(ctx, a));
      }
      }
      CAI_TRY(op_moe_combine(ctx, x, H, s->pair_out, H, s->gates, B, K, H));
    }
  }
  if (s->kv_owner) {
    // prefill helper: only the caches matter, no logits, no argmax, no advance (the host sets the next chunk's rows)
    if (x != s->x) return cai_fail(ctx, CAI_ERR_STATE, "internal: residual buffer parity");
    return CAI_OK;
  }
  if (linear_can_fuse_norm(&m->lm_head, B)) {
    LinearArgs a; a.w = &m->lm_head; a.x = x; a.ldx = H; a.y = s->logits; a.ldy = m->vocab_l; a.batch = B;
    a.norm_gain = m->final_norm; a.norm_eps = c.rms_eps;
    CAI_TRY(linear_launch(ctx, a));
  } else {
    CAI_TRY(op_rmsnorm(ctx, x, H, m->final_norm, s->h, H, B, H, c.rms_eps));
    LinearArgs a; a.w = &m->lm_head; a.x = s->h; a.ldx = H; a.y = s->logits; a.ldy = m->vocab_l; a.batch = B;
    CAI_TRY(linear_launch(ctx, a));
  }
  CAI_TRY(op_argmax(ctx, s->logits, m->vocab_l, B, m->vocab_l, s->amax_idx, s->amax_val, s->amax_part_val, s->amax_part_idx, s->amax_tickets));
  if (m->tp_size > 1) {
    pdl_launch(ctx, pack_argmax_kernel, dim3((B + 127) / 128), dim3(128), 0, (const int32_t*)s->amax_idx, (const float*)s->amax_val, B, m->tp_rank * m->vocab_l, s->amax_pack);
    CAI_LAUNCHED(ctx);
    CAI_TRY(comm_allgather(ctx, s->amax_pack, s->amax_gather, (int64_t)B * 2));
    pdl_launch(ctx, pick_argmax_kernel, dim3((B + 127) / 128), dim3(128), 0, (const float*)s->amax_gather, B, m->tp_size, s->amax_idx);
    CAI_LAUNCHED(ctx);
  }
  if (B > 1024) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "batch above 1024");
  pdl_launch(ctx, advance_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, s->tokens_dev, s->pos_dev, s->len_dev,
             (const int32_t*)s->amax_idx, B, s->trace, s->trace_count, s->trace_cap);
  CAI_LAUNCHED(ctx);
  if (x != s->x) return cai_fail(ctx, CAI_ERR_STATE, "internal: residual buffer parity");
  return CAI_OK;
}

// Runs one step: through the captured CUDA graph when enabled, else eagerly.
static int run_step(cai_session* s) {
  cai_ctx* ctx = s->ctx;
  if (!s->use_graph || s->plan) return enqueue_step(s);     // the persistent step kernel is one launch: a graph adds nothing
  if (!s->graph_exec) {
    const int64_t before = ctx->launches;
    cudaGraph_t graph = nullptr;
    CAI_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    const int st = enqueue_step(s);
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (st != CAI_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "cudaStreamEndCapture -> %s", cudaGetErrorString(e));
    s->graph_kernels = ctx->launches - before;
    ctx->launches = before;
    e = cudaGraphInstantiate(&s->graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { s->graph_exec = nullptr; return cai_fail(ctx, CAI_ERR_CUDA, "cudaGraphInstantiate -> %s", cudaGetErrorString(e)); }
  }
  CAI_CUDA(ctx, cudaGraphLaunch(s->graph_exec, ctx->stream));
  ctx->launches += s->graph_kernels;
  return CAI_OK;
}

static int push_len(cai_session* s) {
  cai_ctx* ctx = s->ctx;
  int32_t* pin = s->io_pinned + 2 * s->batch;
  for (int b = 0; b < s->batch; ++b) pin[b] = s->len_host[(size_t)b];
  CAI_CUDA(ctx, cudaMemcpyAsync(s->len_dev, pin, (size_t)s->batch * 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

// Reports a raised device error word; a step kernel that gave up a wait leaves its barrier words behind, which are
// cleared here so that the session stays usable.
static int session_check(cai_session* s) {
  const int st = cai_check_device_error(s->ctx);
  if (st != CAI_OK && s->plan) {
    char keep[sizeof(s->ctx->err)];
    memcpy(keep, s->ctx->err, sizeof(keep));
    step_plan_reset_sync(s->ctx, s->plan);
    memcpy(s->ctx->err, keep, sizeof(keep));
  }
  return st;
}

static int check_room(cai_session* s, int steps) {
  if (s->evict_window > 0) return CAI_OK;                   // a stream with eviction never fills its cache
  for (int b = 0; b < s->batch; ++b)
    if (s->len_host[(size_t)b] + steps > s->max_ctx)
      return cai_fail(s->ctx, CAI_ERR_STATE, "context full: sequence %d holds %d of %d positions, %d more requested", b,
                      s->len_host[(size_t)b], s->max_ctx, steps);
  return CAI_OK;
}

extern "C" {

int cai_session_destroy(cai_session* s) {
  if (!s) return CAI_ERR_INVALID;
  cudaSetDevice(s->ctx->device);
  cudaStreamSynchronize(s->ctx->stream);
  if (s->wide) { cai_session_destroy(s->wide); s->wide = nullptr; }
  if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
  if (s->plan) step_plan_destroy(s->plan);
  if (s->plan_ts) cudaFree(s->plan_ts);
  if (s->sample_scratch) cudaFree(s->sample_scratch);
  if (s->sample_ids) cudaFree(s->sample_ids);
  if (s->sample_probs) cudaFree(s->sample_probs);
  if (s->sample_u) cudaFree(s->sample_u);
  if (s->ar) comm_ar_destroy(s->ctx, s->ar);
  if (s->kv_owner) { s->k_cache = s->v_cache = nullptr; s->k_scales = s->v_scales = nullptr; }   // borrowed
  void* bufs[] = {s->seq_index_dev, s->k_cache, s->v_cache, s->k_snap, s->v_snap, s->tokens_dev, s->pos_dev, s->len_dev, s->x, s->x_alt, s->h, s->qkv,
                  s->att, s->act, s->gu, s->logits, s->router_logits, s->gates, s->moe_hidden, s->pair_out, s->expert_ids, s->partial,
                  s->amax_idx, s->amax_val, s->amax_part_val, s->amax_part_idx, s->amax_tickets, s->rope_cs, s->amax_pack, s->amax_gather, s->logits_gather, s->trace, s->trace_count, s->prefill_buf,
                  s->tile_expert, s->tile_pairs, s->moe_gu, s->moe_unscale, s->moe_xp,
                  s->ep_pack, s->ep_all, s->ep_gates, s->ep_part, s->ep_mine, s->ep_ids,
                  s->k_scales, s->v_scales, s->k_scales_snap, s->v_scales_snap};
  for (void* p : bufs) if (p) cudaFree(p);
  if (s->io_pinned) cudaFreeHost(s->io_pinned);
  s->m->sessions -= 1;
  delete s;
  return CAI_OK;
}

static int session_create_impl(cai_model* m, int max_ctx, int batch, int kv_type, cai_session* kv_owner, cai_session** out);

int cai_session_create(cai_model* m, int max_ctx, int batch, int kv_type, cai_session** out) {
  return session_create_impl(m, max_ctx, batch, kv_type, nullptr, out);
}

// kv_owner != NULL: a prefill helper whose `batch` rows index into the owner's caches (nothing is allocated for them)
static int session_create_impl(cai_model* m, int max_ctx, int batch, int kv_type, cai_session* kv_owner, cai_session** out) {
  if (!m) return CAI_ERR_INVALID;
  cai_ctx* ctx = m->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_create: null output");
  *out = nullptr;
  if (!m->finalized) return cai_fail(ctx, CAI_ERR_STATE, "call cai_model_finalize before creating sessions");
  if (max_ctx < 1 || batch < 1 || batch > 1024) return cai_fail(ctx, CAI_ERR_INVALID, "max_ctx %d batch %d", max_ctx, batch);
  if (kv_type != CAI_TYPE_F32 && kv_type != CAI_TYPE_I8) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "KV cache type %d: fp32 (0) or int8 (24)", kv_type);
  const cai_llama_config& c = m->cfg;
  const bool kv_int8 = kv_type == CAI_TYPE_I8;
  if (kv_int8 && !attn_int8_supported(m->heads_l, m->kv_heads_l, c.head_dim))
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "the int8 KV cache needs head_dim 64 or 128 and at most 8 query heads per KV head");
  const int cache_seqs = kv_owner ? kv_owner->batch : batch;
  const int ctx_pitch = (max_ctx + 31) & ~31;
  const size_t layer_stride = (size_t)cache_seqs * m->kv_heads_l * ctx_pitch * c.head_dim;
  const size_t scale_stride = (size_t)cache_seqs * m->kv_heads_l * ctx_pitch;
  const size_t cache_bytes = kv_owner ? 0 : layer_stride * (size_t)c.layers * (kv_int8 ? 1 : 4) + (kv_int8 ? scale_stride * (size_t)c.layers * 4 : 0);
  size_t free_b = 0, total_b = 0;
  CAI_CUDA(ctx, cudaMemGetInfo(&free_b, &total_b));
  if (2 * cache_bytes + ((size_t)256 << 20) > free_b)
    return cai_fail(ctx, CAI_ERR_OOM, "KV cache of %zu bytes does not fit in %zu free device bytes", 2 * cache_bytes, free_b);
  cai_session* s = new (std::nothrow) cai_session();
  if (!s) return cai_fail(ctx, CAI_ERR_OOM, "host allocation failed");
  s->m = m; s->ctx = ctx; s->max_ctx = max_ctx; s->batch = batch; s->layer_stride = layer_stride;
  s->ctx_pitch = ctx_pitch;
  s->k_blocked = kv_owner ? kv_owner->k_blocked : (attn_k_blocked_supported(m->heads_l, m->kv_heads_l, c.head_dim) ? 1 : 0);
  s->kv_int8 = kv_int8; s->scale_stride = scale_stride;
  s->len_host.assign((size_t)batch, 0);
  m->sessions += 1;
  const char* ng = getenv("CAI_NO_GRAPH");
  s->use_graph = !(ng && *ng && *ng != '0') && !CAI_CHECKED_BUILD;   // the checked build looks at every launch on its own
  // Programmatic dependent launch pays when the step is a chain of short kernels (the next kernel's CTAs are
  // resident and primed when the previous one drains); on the 32B model, whose kernels each stream > 100 MB, it
  // measured slower. Rule: on when one layer's MLP weights are below 24 M elements.
  s->use_pdl = ctx->pdl_mode >= 0 ? ctx->pdl_mode : (((int64_t)c.hidden * m->inter_l * 3 < ((int64_t)24 << 20)) ? 1 : 0);
  const int B = batch, H = c.hidden, QKVW = m->qw_l + 2 * m->kw_l;
  s->nsplit = attn_nsplit(ctx, B, m->kv_heads_l, max_ctx);
  s->trace_cap = (int64_t)max_ctx * B;
  bool ok = true;
  auto A = [&](void** p, size_t bytes) { if (ok && cudaMalloc(p, bytes ? bytes : 4) != cudaSuccess) { cudaGetLastError(); ok = false; } };
  if (kv_owner) {
    s->kv_owner = kv_owner;
    s->k_cache = kv_owner->k_cache; s->v_cache = kv_owner->v_cache; s->k_scales = kv_owner->k_scales; s->v_scales = kv_owner->v_scales;
    A((void**)&s->seq_index_dev, (size_t)B * 4);
  } else {
    A((void**)&s->k_cache, s->cache_bytes()); A((void**)&s->v_cache, s->cache_bytes());
    if (kv_int8) { A((void**)&s->k_scales, s->scale_bytes()); A((void**)&s->v_scales, s->scale_bytes()); }
  }
  A((void**)&s->tokens_dev, (size_t)B * 4); A((void**)&s->pos_dev, (size_t)B * 4); A((void**)&s->len_dev, (size_t)B * 4);
  A((void**)&s->x, (size_t)B * H * 4); A((void**)&s->x_alt, (size_t)B * H * 4); A((void**)&s->h, (size_t)B * H * 4);
  A((void**)&s->qkv, (size_t)B * QKVW * 4); A((void**)&s->att, (size_t)B * m->qw_l * 4);
  A((void**)&s->act, (size_t)B * (m->inter_l ? m->inter_l : 1) * 4);
  A((void**)&s->logits, (size_t)B * m->vocab_l * 4);
  bool any_split = false;
  for (const LayerW& L : m->layers) any_split = any_split || L.qkv_split || L.gu_split;
  if (((B >= 3 && B <= 64) || any_split) && m->inter_l) A((void**)&s->gu, (size_t)B * 2 * m->inter_l * 4);
  size_t partial_floats = attn_partial_floats(B, m->heads_l, s->nsplit, c.head_dim);
  if (B == 1) {
    // the persistent step kernel deals about one (kv head, context split) item to every SM
    int ns = ctx->sm_count / m->kv_heads_l;
    if (ns > (max_ctx + 31) / 32) ns = (max_ctx + 31) / 32;
    if (ns < 1) ns = 1;
    const size_t need = attn_partial_floats(1, m->heads_l, ns, c.head_dim);
    if (need > partial_floats) partial_floats = need;
  }
  A((void**)&s->partial, partial_floats * 4);
  A((void**)&s->amax_idx, (size_t)B * 4); A((void**)&s->amax_val, (size_t)B * 4);
  A((void**)&s->amax_part_val, (size_t)B * CAI_ARGMAX_CHUNKS * 4); A((void**)&s->amax_part_idx, (size_t)B * CAI_ARGMAX_CHUNKS * 4);
  A((void**)&s->amax_tickets, (size_t)B * 4); A((void**)&s->rope_cs, (size_t)B * c.head_dim * 4);
  A((void**)&s->trace, (size_t)s->trace_cap * 4); A((void**)&s->trace_count, 4);
  if (c.n_experts) {
    A((void**)&s->router_logits, (size_t)B * c.n_experts * 4); A((void**)&s->gates, (size_t)B * c.top_k * 4);
    A((void**)&s->expert_ids, (size_t)B * c.top_k * 4);
    const int Bm = B * m->ep_size;             // sequences whose pairs this rank may have to run (all ranks' under expert parallelism)
    const int pairs = Bm * c.top_k;
    A((void**)&s->moe_hidden, (size_t)pairs * c.moe_inter * 4); A((void**)&s->pair_out, (size_t)pairs * H * 4);
    {
      // Grouped tensor-core path when an expert sees two or more pairs on average (otherwise most tiles would hold one
      // pair and the per-pair GEMV is the better kernel), quantized experts, whole 32-blocks. Expert parallelism
      // always takes it.
      const QWeight& gu = m->layers[0].exp_gu[(size_t)m->expert_lo()];
      const bool quant = gu.type == CAI_TYPE_Q8_0 || gu.type == CAI_TYPE_Q4_0;
      const char* off = getenv("CAI_MOE_GROUPED");
      const bool can = quant && pairs <= 4096 && c.n_experts <= 1024 && H % 32 == 0 && c.moe_inter % 32 == 0;
      if (m->ep_size > 1 && !can) {
        cai_session_destroy(s);
        return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "expert parallelism needs Q8_0 / Q4_0 experts, at most 4096 (token, expert) pairs per step and 32-aligned widths");
      }
      if (can && (m->ep_size > 1 || (pairs >= 2 * c.n_experts && !(off && *off == '0')))) {
        const int local_experts = c.n_experts / m->ep_size;
        s->moe_tiles = pairs / 16 + (pairs < local_experts ? pairs : local_experts) + 1;  // sum over experts of ceil(count / 16) is below this
        const size_t tile_bytes = gemm_tc_group_tile_bytes(H > c.moe_inter ? H : c.moe_inter);
        A((void**)&s->tile_expert, (size_t)s->moe_tiles * 4); A((void**)&s->tile_pairs, (size_t)s->moe_tiles * 16 * 4);
        A((void**)&s->moe_gu, (size_t)pairs * 2 * c.moe_inter * 4);
        A((void**)&s->moe_unscale, (size_t)s->moe_tiles * 16 * 4); A(&s->moe_xp, (size_t)s->moe_tiles * tile_bytes);
      }
      if (m->ep_size > 1) {
        const size_t W = ((size_t)H + 2 * (size_t)c.top_k + 3) & ~(size_t)3;       // packed row: h | ids | gates, padded to 16 bytes
        A((void**)&s->ep_pack, (size_t)B * W * 4); A((void**)&s->ep_all, (size_t)Bm * W * 4);
        A((void**)&s->ep_ids, (size_t)pairs * 4); A((void**)&s->ep_gates, (size_t)pairs * 4);
        A((void**)&s->ep_part, (size_t)Bm * H * 4); A((void**)&s->ep_mine, (size_t)B * H * 4);
      }
    }
  }
  if (m->tp_size > 1) {
    A((void**)&s->amax_pack, (size_t)B * 2 * 4); A((void**)&s->amax_gather, (size_t)m->tp_size * B * 2 * 4);
    A((void**)&s->logits_gather, (size_t)m->tp_size * B * m->vocab_l * 4);
  }
  if (ok && !kv_owner && m->tp_size > 1 && ((int64_t)B * H) % 4 == 0) {
    // collective: every rank creates its session at the same point
    // slots: one per call site of the per-operator path; the step kernel's row exchange needs 4 x world rows of pairs
    // and one more slot for the argmax exchange
    const int sites = (2 * c.layers + 1 > 4 * m->tp_size + 1) ? 2 * c.layers + 1 : 4 * m->tp_size + 1;
    if (comm_ar_create(ctx, sites, (int64_t)B * H, &s->ar) != CAI_OK) ok = false;
  }
  if (ok && !kv_owner && m->ep_size > 1 && c.n_experts > 0 && (H % 4) == 0) {
    // collective: the expert-parallel dispatch / combine over peer memory, one slot per exchange of a step
    // (CAI_EP_EXCHANGE=nccl, or peers that cannot be mapped: the library's all-gather and reduce-scatter instead)
    const char* em = getenv("CAI_EP_EXCHANGE");
    if (!(em && !strcmp(em, "nccl"))) {
      const int W = (H + 2 * c.top_k + 3) & ~3;
      int64_t elems = (int64_t)B * m->ep_size * H;
      if ((int64_t)B * W > elems) elems = (int64_t)B * W;
      if (comm_ar_create(ctx, 2 * c.layers, (elems + 3) & ~(int64_t)3, &s->ar) != CAI_OK) ok = false;
    }
  }
  if (ok && cudaMallocHost((void**)&s->io_pinned, (size_t)4 * B * 4) != cudaSuccess) { cudaGetLastError(); ok = false; }
  if (ok && B >= 3 && B <= 64) {
    // the tensor-core GEMM's activation buffer must exist before a step is captured into a graph
    int64_t kmax = H;
    if (m->qw_l > kmax) kmax = m->qw_l;
    if (m->inter_l > kmax) kmax = m->inter_l;
    if (gemm_tc_reserve(ctx, kmax, B) != CAI_OK) ok = false;
  }
  if (!ok) { cai_session_destroy(s); return cai_fail(ctx, CAI_ERR_OOM, "session buffers do not fit on the device"); }
  CAI_CUDA(ctx, cudaMemsetAsync(s->len_dev, 0, (size_t)B * 4, ctx->stream));
  CAI_CUDA(ctx, cudaMemsetAsync(s->pos_dev, 0, (size_t)B * 4, ctx->stream));
  CAI_CUDA(ctx, cudaMemsetAsync(s->tokens_dev, 0, (size_t)B * 4, ctx->stream));
  CAI_CUDA(ctx, cudaMemsetAsync(s->trace_count, 0, 4, ctx->stream));
  CAI_CUDA(ctx, cudaMemsetAsync(s->amax_tickets, 0, (size_t)B * 4, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  // Which sessions take the persistent step kernel when nothing forces it (CAI_STEP_KERNEL=1 / 0): a phase of that
  // kernel costs 6-10 us whatever it streams (grid barrier, staging, the slowest warp), a launch of the per-operator
  // path ~5 us; measured on B200, the step kernel wins where a layer's products are large (Qwen2.5-32B shape: 9.07 against
  // 9.96 ms per step) and loses on small layers (Qwen2.5-0.5B shape: 0.95 against 0.78 ms). Rule: on when one layer's
  // MLP weights on this rank reach 24 M elements, and for every tensor-parallel session (there the alternative pays two
  // extra launches per layer for the sums over the ranks).
  const int step_mode = env_int("CAI_STEP_KERNEL", -1);
  const bool step_auto = ((int64_t)c.hidden * m->inter_l * 3 >= ((int64_t)24 << 20)) || m->tp_size > 1;
  if (B == 1 && !any_split && !kv_owner && !kv_int8 && !c.n_experts && !c.qk_norm && (m->tp_size == 1 || s->ar) && (step_mode == 1 || (step_mode < 0 && step_auto))) {
    // the whole step as one persistent kernel when the model is inside what it covers; otherwise (status
    // CAI_ERR_UNSUPPORTED) the session keeps one launch per operator
    StepSetup u;
    u.layers = c.layers; u.hidden = H; u.q_heads = m->heads_l; u.kv_heads = m->kv_heads_l; u.head_dim = c.head_dim;
    u.inter = m->inter_l; u.vocab = m->vocab_l; u.max_ctx = ctx_pitch; u.k_blocked = s->k_blocked; u.rms_eps = c.rms_eps;
    u.embed = &m->embed; u.lm_head = &m->lm_head; u.final_norm = m->final_norm; u.theta = m->theta;
    u.layer.resize((size_t)c.layers);
    for (int l = 0; l < c.layers; ++l) {
      LayerW& L = m->layers[(size_t)l];
      StepLayerSetup& d = u.layer[(size_t)l];
      d.wqkv = &L.wqkv; d.wo = &L.wo; d.wgu = &L.wgu; d.wdown = &L.wdown; d.attn_norm = L.attn_norm; d.ffn_norm = L.ffn_norm;
      d.k_cache = s->k_cache + (size_t)l * s->layer_stride; d.v_cache = s->v_cache + (size_t)l * s->layer_stride;
    }
    u.tokens = s->tokens_dev; u.pos = s->pos_dev; u.len = s->len_dev;
    u.xres = s->x; u.qbuf = s->qkv; u.att = s->att; u.act = s->act; u.logits = s->logits; u.partial = s->partial;
    u.partial_floats = partial_floats;
    u.amax_idx = s->amax_idx; u.amax_val = s->amax_val; u.trace = s->trace; u.trace_count = s->trace_count; u.trace_cap = s->trace_cap;
    u.ar = s->ar; u.tp_rank = m->tp_rank; u.tp_world = m->tp_size; u.vocab_offset = m->tp_rank * m->vocab_l;
    const int st = step_plan_create(ctx, u, &s->plan);
    if (st != CAI_OK && st != CAI_ERR_UNSUPPORTED) { cai_session_destroy(s); return cai_fail(ctx, st, "step kernel set-up failed"); }
  }
  *out = s;
  return CAI_OK;
}

int cai_session_reset(cai_session* s, int seq) {
  if (!s) return CAI_ERR_INVALID;
  CAI_TRY(cai_bind(s->ctx));
  if (seq < -1 || seq >= s->batch) return cai_fail(s->ctx, CAI_ERR_INVALID, "sequence %d of %d", seq, s->batch);
  for (int b = 0; b < s->batch; ++b) if (seq < 0 || seq == b) s->len_host[(size_t)b] = 0;
  return push_len(s);
}

int cai_session_truncate(cai_session* s, int seq, int committed_len) {
  if (!s) return CAI_ERR_INVALID;
  CAI_TRY(cai_bind(s->ctx));
  if (seq < 0 || seq >= s->batch) return cai_fail(s->ctx, CAI_ERR_INVALID, "sequence %d of %d", seq, s->batch);
  if (committed_len < 0 || committed_len > s->len_host[(size_t)seq])
    return cai_fail(s->ctx, CAI_ERR_INVALID, "truncate to %d outside the committed prefix of %d", committed_len, s->len_host[(size_t)seq]);
  if (s->evict_window > 0 && s->len_host[(size_t)seq] > s->evict_sinks + s->evict_window && committed_len != s->len_host[(size_t)seq])
    return cai_fail(s->ctx, CAI_ERR_STATE, "truncate after eviction has dropped rows: the rows a shorter prefix needs are gone");
  s->len_host[(size_t)seq] = committed_len;
  return push_len(s);
}

int cai_session_fill_for_benchmark(cai_session* s, int n_rows) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (s->kv_owner) return cai_fail(ctx, CAI_ERR_STATE, "cai_session_fill_for_benchmark: not on a prefill helper");
  if (n_rows < 0 || n_rows > s->max_ctx) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_fill_for_benchmark: %d rows of %d", n_rows, s->max_ctx);
  CAI_CUDA(ctx, cudaMemsetAsync(s->k_cache, 0, s->cache_bytes(), ctx->stream));
  CAI_CUDA(ctx, cudaMemsetAsync(s->v_cache, 0, s->cache_bytes(), ctx->stream));
  if (s->kv_int8) {
    // scale 1 with zero codes: the row format's own encoding of an all-zero row
    std::vector<float> ones(1 << 20, 1.0f);
    const size_t total = s->scale_stride * (size_t)s->m->cfg.layers;
    for (size_t at = 0; at < total; at += ones.size()) {
      const size_t nn = total - at < ones.size() ? total - at : ones.size();
      CAI_CUDA(ctx, cudaMemcpyAsync(s->k_scales + at, ones.data(), nn * 4, cudaMemcpyHostToDevice, ctx->stream));
      CAI_CUDA(ctx, cudaMemcpyAsync(s->v_scales + at, ones.data(), nn * 4, cudaMemcpyHostToDevice, ctx->stream));
      CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
  }
  for (auto& l : s->len_host) l = n_rows;
  return push_len(s);
}

// A change of what the steps see invalidates anything captured with the old parameters.
static void session_drop_captured(cai_session* s) {
  if (s->graph_exec) { cudaGraphExecDestroy(s->graph_exec); s->graph_exec = nullptr; }
  if (s->plan) { step_plan_destroy(s->plan); s->plan = nullptr; }      // the persistent step kernel attends over the whole cache
  if (s->wide) { cai_session_destroy(s->wide); s->wide = nullptr; }
}

int cai_session_enable_eviction(cai_session* s, int sink_tokens, int recent_window) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (s->kv_owner) return cai_fail(ctx, CAI_ERR_STATE, "not on a prefill helper");
  if (sink_tokens < 0 || recent_window < 0 || (recent_window == 0 && sink_tokens != 0) || sink_tokens + recent_window > s->max_ctx)
    return cai_fail(ctx, CAI_ERR_INVALID, "eviction with %d sinks + %d recent rows in a cache of %d", sink_tokens, recent_window, s->max_ctx);
  const int cap = recent_window > 0 ? sink_tokens + recent_window : s->max_ctx;
  for (int l : s->len_host)
    if (l > cap || (s->evict_window > 0 && l > s->evict_sinks + s->evict_window))
      return cai_fail(ctx, CAI_ERR_STATE, "the policy can change only while every sequence holds no more rows than it keeps");
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  session_drop_captured(s);
  s->evict_sinks = sink_tokens; s->evict_window = recent_window;
  return CAI_OK;
}

int cai_session_set_window(cai_session* s, int window) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (s->kv_owner) return cai_fail(ctx, CAI_ERR_STATE, "not on a prefill helper");
  if (window < 0) return cai_fail(ctx, CAI_ERR_INVALID, "window %d", window);
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  session_drop_captured(s);
  s->window = window;
  return CAI_OK;
}

int cai_session_cache_len(cai_session* s, int seq, int* out_len) {
  if (!s || !out_len) return CAI_ERR_INVALID;
  if (seq < 0 || seq >= s->batch) return cai_fail(s->ctx, CAI_ERR_INVALID, "sequence %d of %d", seq, s->batch);
  *out_len = s->len_host[(size_t)seq];
  return CAI_OK;
}

static int stage_inputs(cai_session* s, const int32_t* tokens_host, const int32_t* abs_pos_host) {
  cai_ctx* ctx = s->ctx;
  const int B = s->batch;
  const int vocab = s->m->cfg.vocab;
  for (int b = 0; b < B; ++b) {
    if (tokens_host[b] < 0 || tokens_host[b] >= vocab) return cai_fail(ctx, CAI_ERR_INVALID, "token id %d outside the vocabulary of %d", tokens_host[b], vocab);
    s->io_pinned[b] = tokens_host[b];
    s->io_pinned[B + b] = abs_pos_host ? abs_pos_host[b] : s->len_host[(size_t)b];
  }
  CAI_CUDA(ctx, cudaMemcpyAsync(s->tokens_dev, s->io_pinned, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaMemcpyAsync(s->pos_dev, s->io_pinned + B, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
  return CAI_OK;
}

int cai_session_step(cai_session* s, const int32_t* tokens_host, const int32_t* abs_pos_host, float* logits_out_host,
                     int32_t* argmax_out_host) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  cai_model* m = s->m;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_step: null tokens");
  CAI_TRY(check_room(s, 1));
  CAI_TRY(stage_inputs(s, tokens_host, abs_pos_host));
  CAI_TRY(run_step(s));
  for (auto& l : s->len_host) l += 1;
  const int B = s->batch, Vl = m->vocab_l, V = m->cfg.vocab;
  if (logits_out_host) {
    if (m->tp_size == 1) {
      CAI_CUDA(ctx, cudaMemcpyAsync(logits_out_host, s->logits, (size_t)B * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
    } else {
      CAI_TRY(comm_allgather(ctx, s->logits, s->logits_gather, (int64_t)B * Vl));
      s->host_gather.resize((size_t)m->tp_size * B * Vl);
      CAI_CUDA(ctx, cudaMemcpyAsync(s->host_gather.data(), s->logits_gather, s->host_gather.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
  }
  if (argmax_out_host) CAI_CUDA(ctx, cudaMemcpyAsync(argmax_out_host, s->amax_idx, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  CAI_TRY(session_check(s));
  if (logits_out_host && m->tp_size > 1) {
    for (int r = 0; r < m->tp_size; ++r)
      for (int b = 0; b < B; ++b)
        memcpy(logits_out_host + (size_t)b * V + (size_t)r * Vl, s->host_gather.data() + ((size_t)r * B + b) * Vl, (size_t)Vl * 4);
  }
  return CAI_OK;
}

int cai_session_decode_greedy(cai_session* s, const int32_t* tokens_host, int n_steps, int32_t* out_tokens_host) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host || n_steps < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_decode_greedy: bad argument");
  CAI_TRY(check_room(s, n_steps));
  CAI_TRY(stage_inputs(s, tokens_host, nullptr));
  CAI_CUDA(ctx, cudaMemsetAsync(s->trace_count, 0, 4, ctx->stream));
  for (int i = 0; i < n_steps; ++i) CAI_TRY(run_step(s));
  for (auto& l : s->len_host) l += n_steps;
  if (out_tokens_host)
    CAI_CUDA(ctx, cudaMemcpyAsync(out_tokens_host, s->trace, (size_t)n_steps * s->batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return session_check(s);
}

static int sample_ensure(cai_session* s) {
  cai_ctx* ctx = s->ctx;
  if (s->m->tp_size > 1) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "device sampling needs the whole logits row on one GPU (tensor-parallel sessions shard the vocabulary)");
  if (s->sample_scratch) return CAI_OK;
  const int B = s->batch;
  CAI_CUDA(ctx, cudaMalloc((void**)&s->sample_scratch, (size_t)sample_scratch_floats(B) * 4));
  CAI_CUDA(ctx, cudaMalloc((void**)&s->sample_ids, (size_t)B * 64 * 4));
  CAI_CUDA(ctx, cudaMalloc((void**)&s->sample_probs, (size_t)B * 64 * 4));
  CAI_CUDA(ctx, cudaMalloc((void**)&s->sample_u, (size_t)B * 4));
  return CAI_OK;
}

int cai_session_step_topk(cai_session* s, const int32_t* tokens_host, const int32_t* abs_pos_host, int k, float temperature,
                          int32_t* ids_out_host, float* probs_out_host) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host || !ids_out_host || !probs_out_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_step_topk: null argument");
  CAI_TRY(sample_ensure(s));
  CAI_TRY(check_room(s, 1));
  CAI_TRY(stage_inputs(s, tokens_host, abs_pos_host));
  CAI_TRY(run_step(s));
  for (auto& l : s->len_host) l += 1;
  CAI_TRY(sample_launch(ctx, s->logits, s->m->vocab_l, s->batch, s->m->vocab_l, k, temperature, 0.f, 0ull, nullptr, s->sample_scratch,
                        s->sample_ids, s->sample_probs, nullptr, nullptr, nullptr, 0, nullptr));
  CAI_CUDA(ctx, cudaMemcpyAsync(ids_out_host, s->sample_ids, (size_t)s->batch * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaMemcpyAsync(probs_out_host, s->sample_probs, (size_t)s->batch * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return session_check(s);
}

int cai_session_decode_sampled(cai_session* s, const int32_t* tokens_host, int n_steps, const cai_sampling* opt, const float* uniforms_host,
                               int32_t* out_tokens_host) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host || n_steps < 1 || !opt) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_decode_sampled: bad argument");
  if (opt->top_k < 1 || opt->top_k > 64) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "cai_session_decode_sampled: top_k %d outside 1..64", opt->top_k);
  CAI_TRY(sample_ensure(s));
  CAI_TRY(check_room(s, n_steps));
  CAI_TRY(stage_inputs(s, tokens_host, nullptr));
  CAI_CUDA(ctx, cudaMemsetAsync(s->trace_count, 0, 4, ctx->stream));
  for (int i = 0; i < n_steps; ++i) {
    if (uniforms_host) {
      CAI_CUDA(ctx, cudaMemcpyAsync(s->sample_u, uniforms_host + (size_t)i * s->batch, (size_t)s->batch * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    CAI_TRY(run_step(s));                      // forward + greedy advance; the draw below replaces the token it chose
    CAI_TRY(sample_launch(ctx, s->logits, s->m->vocab_l, s->batch, s->m->vocab_l, opt->top_k, opt->temperature, opt->top_p, opt->seed,
                          uniforms_host ? s->sample_u : nullptr, s->sample_scratch, nullptr, nullptr, s->tokens_dev, s->trace, s->trace_count,
                          s->trace_cap, nullptr));
    if (uniforms_host) CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));     // the pageable source row is reused by nothing, but keep it simple
  }
  for (auto& l : s->len_host) l += n_steps;
  if (out_tokens_host)
    CAI_CUDA(ctx, cudaMemcpyAsync(out_tokens_host, s->trace, (size_t)n_steps * s->batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return session_check(s);
}

int cai_session_prefill(cai_session* s, const int32_t* tokens_host, int n_tokens) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host || n_tokens < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_prefill: bad argument");
  CAI_TRY(check_room(s, n_tokens));
  const int B = s->batch, vocab = s->m->cfg.vocab;
  const int64_t need = (int64_t)n_tokens * B;
  if (s->prefill_cap < need) {
    if (s->prefill_buf) cudaFree(s->prefill_buf);
    s->prefill_buf = nullptr; s->prefill_cap = 0;
    CAI_CUDA(ctx, cudaMalloc((void**)&s->prefill_buf, (size_t)need * 4));
    s->prefill_cap = need;
  }
  for (int64_t i = 0; i < need; ++i)
    if (tokens_host[i] < 0 || tokens_host[i] >= vocab) return cai_fail(ctx, CAI_ERR_INVALID, "token id %d outside the vocabulary of %d", tokens_host[i], vocab);
  // Chunked prefill: C consecutive positions of every sequence per step (B x C <= 64 rows, the tensor-core GEMM's
  // batch), through a helper session that appends to and attends over THIS session's caches: row (b, i) of a chunk is
  // position len[b] + i of sequence b and sees the rows before it, the chunk's own earlier rows included. The
  // reference prefills one token at a time (neural/neuralchatengine.pas:1466-1470); the caches come out the same
  // up to the arithmetic of the batched kernels (tests compare the two). CAI_PREFILL_CHUNK=0 turns it off. What is
  // left over after the whole chunks goes through the token-at-a-time loop below.
  int done = 0;
  {
    const char* off = getenv("CAI_PREFILL_CHUNK");
    const int C = (B <= 32) ? 64 / B : 0;
    if (C >= 2 && n_tokens >= C && !(off && *off == '0') && !s->kv_owner && !s->evict_window) {
      if (!s->wide) {
        cai_session* w = nullptr;
        const int st = session_create_impl(s->m, s->max_ctx, B * C, s->kv_int8 ? CAI_TYPE_I8 : CAI_TYPE_F32, s, &w);
        if (st == CAI_OK) { s->wide = w; s->wide_chunk = C; }
        else if (st != CAI_ERR_OOM) return st;             // no room for the helper: keep the token-at-a-time path
      }
      cai_session* w = s->wide;
      if (w) {
        const int R = B * C;
        for (; done + C <= n_tokens; done += C) {
          int32_t* pin = w->io_pinned;
          for (int b = 0; b < B; ++b)
            for (int i = 0; i < C; ++i) {
              const int r = b * C + i, at = s->len_host[(size_t)b] + done + i;
              pin[r] = tokens_host[(size_t)b * n_tokens + done + i];
              pin[R + r] = at;                               // absolute position = cache slot during prefill
              pin[2 * R + r] = at;                           // rows of the sequence cached before this one
              pin[3 * R + r] = b;
            }
          CAI_CUDA(ctx, cudaMemcpyAsync(w->tokens_dev, pin, (size_t)R * 4, cudaMemcpyHostToDevice, ctx->stream));
          CAI_CUDA(ctx, cudaMemcpyAsync(w->pos_dev, pin + R, (size_t)R * 4, cudaMemcpyHostToDevice, ctx->stream));
          CAI_CUDA(ctx, cudaMemcpyAsync(w->len_dev, pin + 2 * R, (size_t)R * 4, cudaMemcpyHostToDevice, ctx->stream));
          CAI_CUDA(ctx, cudaMemcpyAsync(w->seq_index_dev, pin + 3 * R, (size_t)R * 4, cudaMemcpyHostToDevice, ctx->stream));
          CAI_TRY(run_step(w));
          CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // the pinned rows are rewritten for the next chunk
        }
        for (auto& l : s->len_host) l += done;
        CAI_TRY(push_len(s));
        if (done == n_tokens) return session_check(s);
      }
    }
  }
  tokens_host += done;                                       // column offset: rows keep the stride n_tokens
  const int n_left = n_tokens - done;
  // step-major copy: row i holds the i-th token of every sequence
  std::vector<int32_t> stepmajor((size_t)need);
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < n_left; ++i) stepmajor[(size_t)i * B + b] = tokens_host[(size_t)b * n_tokens + i];
  CAI_CUDA(ctx, cudaMemcpyAsync(s->prefill_buf, stepmajor.data(), (size_t)n_left * B * 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  std::vector<int32_t> first(stepmajor.begin(), stepmajor.begin() + B);
  CAI_TRY(stage_inputs(s, first.data(), nullptr));
  for (int i = 0; i < n_left; ++i) {
    CAI_CUDA(ctx, cudaMemcpyAsync(s->tokens_dev, s->prefill_buf + (size_t)i * B, (size_t)B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    CAI_TRY(run_step(s));
  }
  for (auto& l : s->len_host) l += n_left;
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return session_check(s);
}

int cai_session_profile(cai_session* s, const int32_t* tokens_host, int n_steps, float* out_ms, int64_t* out_launches) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host || n_steps < 1 || !out_ms || !out_launches) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_profile: bad argument");
  CAI_TRY(check_room(s, n_steps));
  CAI_TRY(stage_inputs(s, tokens_host, nullptr));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int f = 0; f < FAM_COUNT; ++f) { out_ms[f] = 0.f; out_launches[f] = 0; }
  if (s->plan) {
    // persistent step kernel: CTA 0 stamps the global timer at every phase boundary; a phase's time is the span
    // between two stamps, booked to the family of the phase that ended (products, attention, exchanges, the rest)
    const int tl = step_plan_trace_len(s->plan);
    if (!s->plan_ts) CAI_CUDA(ctx, cudaMalloc((void**)&s->plan_ts, (size_t)tl * 8));
    std::vector<unsigned long long> ts((size_t)tl);
    for (int i = 0; i < n_steps; ++i) {
      CAI_CUDA(ctx, cudaMemsetAsync(s->plan_ts, 0, 8, ctx->stream));
      CAI_TRY(step_plan_enqueue(ctx, s->plan, s->plan_ts));
      CAI_CUDA(ctx, cudaMemcpyAsync(ts.data(), s->plan_ts, (size_t)tl * 8, cudaMemcpyDeviceToHost, ctx->stream));
      CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      const int n = (int)ts[0];
      unsigned long long prev = ts[1];
      for (int k = 1; k < n && 2 + 2 * k < tl; ++k) {
        const int f = (int)ts[(size_t)(2 + 2 * k)];
        if (f < 0 || f >= FAM_COUNT) continue;               // stamps inside a phase
        out_ms[f] += (float)((double)(ts[(size_t)(1 + 2 * k)] - prev) * 1e-6);
        out_launches[f] += 1;
        prev = ts[(size_t)(1 + 2 * k)];
      }
    }
    for (auto& l : s->len_host) l += n_steps;
    return session_check(s);
  }
  ctx->prof_n = 0;
  ctx->prof_on = 1;
  int st = cai_prof_mark(ctx, FAM_OTHER);     // origin event
  for (int i = 0; i < n_steps && st == CAI_OK; ++i) st = enqueue_step(s);   // eager launches, one event after each
  ctx->prof_on = 0;
  if (st != CAI_OK) return st;
  for (auto& l : s->len_host) l += n_steps;
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int i = 1; i < ctx->prof_n; ++i) {
    float ms = 0.f;
    CAI_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->prof_events[i - 1], ctx->prof_events[i]));
    const int f = ctx->prof_family[i];
    out_ms[f] += ms;
    out_launches[f] += 1;
  }
  return session_check(s);
}

int cai_session_snapshot(cai_session* s) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  const size_t bytes = s->cache_bytes(), sbytes = s->kv_int8 ? s->scale_bytes() : 0;
  if (!s->k_snap) {
    size_t free_b = 0, total_b = 0;
    CAI_CUDA(ctx, cudaMemGetInfo(&free_b, &total_b));
    if (2 * (bytes + sbytes) + ((size_t)64 << 20) > free_b) return cai_fail(ctx, CAI_ERR_OOM, "snapshot of %zu bytes does not fit", 2 * (bytes + sbytes));
    CAI_CUDA(ctx, cudaMalloc((void**)&s->k_snap, bytes));
    CAI_CUDA(ctx, cudaMalloc((void**)&s->v_snap, bytes));
    if (sbytes) {
      CAI_CUDA(ctx, cudaMalloc((void**)&s->k_scales_snap, sbytes));
      CAI_CUDA(ctx, cudaMalloc((void**)&s->v_scales_snap, sbytes));
    }
  }
  CAI_CUDA(ctx, cudaMemcpyAsync(s->k_snap, s->k_cache, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaMemcpyAsync(s->v_snap, s->v_cache, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  if (sbytes) {
    CAI_CUDA(ctx, cudaMemcpyAsync(s->k_scales_snap, s->k_scales, sbytes, cudaMemcpyDeviceToDevice, ctx->stream));
    CAI_CUDA(ctx, cudaMemcpyAsync(s->v_scales_snap, s->v_scales, sbytes, cudaMemcpyDeviceToDevice, ctx->stream));
  }
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  s->len_snap = s->len_host;
  s->have_snap = true;
  return CAI_OK;
}

int cai_session_restore(cai_session* s) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!s->have_snap) return cai_fail(ctx, CAI_ERR_STATE, "no snapshot to restore");
  const size_t bytes = s->cache_bytes();
  CAI_CUDA(ctx, cudaMemcpyAsync(s->k_cache, s->k_snap, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaMemcpyAsync(s->v_cache, s->v_snap, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  if (s->kv_int8) {
    CAI_CUDA(ctx, cudaMemcpyAsync(s->k_scales, s->k_scales_snap, s->scale_bytes(), cudaMemcpyDeviceToDevice, ctx->stream));
    CAI_CUDA(ctx, cudaMemcpyAsync(s->v_scales, s->v_scales_snap, s->scale_bytes(), cudaMemcpyDeviceToDevice, ctx->stream));
  }
  s->len_host = s->len_snap;
  return push_len(s);
}

int cai_session_logits_dev(cai_session* s, const float** out_dev) {
  if (!s || !out_dev) return CAI_ERR_INVALID;
  *out_dev = s->logits;
  return CAI_OK;
}

int cai_session_step_trace(cai_session* s, const int32_t* tokens_host, int64_t* out_ns, int32_t* out_family, int cap, int* out_n) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!tokens_host || !out_ns || !out_family || !out_n || cap < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_step_trace: bad argument");
  if (!s->plan) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "cai_session_step_trace: the session does not run the persistent step kernel");
  CAI_TRY(check_room(s, 1));
  CAI_TRY(stage_inputs(s, tokens_host, nullptr));
  const int tl = step_plan_trace_len(s->plan);
  if (!s->plan_ts) CAI_CUDA(ctx, cudaMalloc((void**)&s->plan_ts, (size_t)tl * 8));
  std::vector<unsigned long long> ts((size_t)tl);
  CAI_CUDA(ctx, cudaMemsetAsync(s->plan_ts, 0, 8, ctx->stream));
  CAI_TRY(step_plan_enqueue(ctx, s->plan, s->plan_ts));
  CAI_CUDA(ctx, cudaMemcpyAsync(ts.data(), s->plan_ts, (size_t)tl * 8, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto& l : s->len_host) l += 1;
  int n = (int)ts[0];
  if (2 + 2 * (n - 1) >= tl) n = (tl - 1) / 2;
  if (n > cap) n = cap;
  for (int k = 0; k < n; ++k) {
    out_ns[k] = (int64_t)(ts[(size_t)(1 + 2 * k)] - ts[1]);
    out_family[k] = (int32_t)ts[(size_t)(2 + 2 * k)];
  }
  *out_n = n;
  return session_check(s);
}

int cai_session_read_kv_row(cai_session* s, int layer, int seq, int kv_head, int pos, float* k_out_host, float* v_out_host,
                            int8_t* k_codes_host, int8_t* v_codes_host, float* scales_host) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  cai_session* o = s->kv_owner ? s->kv_owner : s;
  const cai_llama_config& c = s->m->cfg;
  const int hd = c.head_dim;
  if (layer < 0 || layer >= c.layers || seq < 0 || seq >= o->batch || kv_head < 0 || kv_head >= s->m->kv_heads_l || pos < 0 ||
      pos >= o->len_host[(size_t)seq])
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_read_kv_row: layer %d sequence %d head %d position %d outside the cached rows", layer, seq, kv_head, pos);
  if (o->evict_window > 0 && o->len_host[(size_t)seq] > o->evict_sinks + o->evict_window) {
    // rows live as sinks + a ring: positions between the sinks and the recent window are gone
    if (pos >= o->evict_sinks && pos < o->len_host[(size_t)seq] - o->evict_window)
      return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_read_kv_row: position %d was evicted", pos);
    if (pos >= o->evict_sinks) pos = o->evict_sinks + (pos - o->evict_sinks) % o->evict_window;
  }
  const size_t head0 = (size_t)layer * o->layer_stride + ((size_t)seq * s->m->kv_heads_l + kv_head) * (size_t)o->ctx_pitch * hd;
  const size_t row0 = head0 + (size_t)pos * hd;
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (o->kv_int8) {
    if (!k_codes_host || !v_codes_host || !scales_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_read_kv_row: the int8 cache needs code and scale outputs");
    const size_t srow = (size_t)layer * o->scale_stride + ((size_t)seq * s->m->kv_heads_l + kv_head) * (size_t)o->ctx_pitch + pos;
    if (o->k_blocked) {
      const int8_t* blk = (const int8_t*)o->k_cache + head0 + (size_t)(pos >> 5) * 32 * hd + (size_t)(pos & 31) * 16;
      CAI_CUDA(ctx, cudaMemcpy2D(k_codes_host, 16, blk, 32 * 16, 16, (size_t)(hd / 16), cudaMemcpyDeviceToHost));
    } else {
      CAI_CUDA(ctx, cudaMemcpy(k_codes_host, (const int8_t*)o->k_cache + row0, (size_t)hd, cudaMemcpyDeviceToHost));
    }
    CAI_CUDA(ctx, cudaMemcpy(v_codes_host, (const int8_t*)o->v_cache + row0, (size_t)hd, cudaMemcpyDeviceToHost));
    CAI_CUDA(ctx, cudaMemcpy(scales_host, o->k_scales + srow, 4, cudaMemcpyDeviceToHost));
    CAI_CUDA(ctx, cudaMemcpy(scales_host + 1, o->v_scales + srow, 4, cudaMemcpyDeviceToHost));
    for (int d = 0; d < hd; ++d) {
      if (k_out_host) k_out_host[d] = scales_host[0] * (float)k_codes_host[d];
      if (v_out_host) v_out_host[d] = scales_host[1] * (float)v_codes_host[d];
    }
    return CAI_OK;
  }
  if (!k_out_host || !v_out_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_session_read_kv_row: null output");
  if (o->k_blocked) {
    // piece p (4 channels) of position pos: float offset (p * 32 + pos % 32) * 4 inside the position's 32-row block
    const float* blk = o->k_cache + head0 + (size_t)(pos >> 5) * 32 * hd + (size_t)(pos & 31) * 4;
    CAI_CUDA(ctx, cudaMemcpy2D(k_out_host, 16, blk, 32 * 16, 16, (size_t)(hd / 4), cudaMemcpyDeviceToHost));
  } else {
    CAI_CUDA(ctx, cudaMemcpy(k_out_host, o->k_cache + row0, (size_t)hd * 4, cudaMemcpyDeviceToHost));
  }
  CAI_CUDA(ctx, cudaMemcpy(v_out_host, o->v_cache + row0, (size_t)hd * 4, cudaMemcpyDeviceToHost));
  if (scales_host) { scales_host[0] = 1.f; scales_host[1] = 1.f; }
  return CAI_OK;
}

int cai_session_uses_step_kernel(cai_session* s, int* out_flag) {
  if (!s || !out_flag) return CAI_ERR_INVALID;
  *out_flag = s->plan ? 1 : 0;
  return CAI_OK;
}

int cai_session_last_kv_bytes(cai_session* s, int64_t* out_bytes) {
  if (!s || !out_bytes) return CAI_ERR_INVALID;
  int64_t rows = 0;
  for (int l : s->len_host) {
    int live = l;
    if (s->evict_window > 0 && live > s->evict_sinks + s->evict_window) live = s->evict_sinks + s->evict_window;
    else if (s->window > 0 && live > s->window) live = s->window;
    rows += live;
  }
  // per cached row and layer: K and V, head_dim values (4 bytes, or 1 byte + a 4-byte scale per head in the int8 cache)
  const int64_t per_row = s->kv_int8 ? (int64_t)s->m->kw_l + 4 * (int64_t)s->m->kv_heads_l : (int64_t)s->m->kw_l * 4;
  *out_bytes = rows * 2 * per_row * (int64_t)s->m->cfg.layers;
  return CAI_OK;
}

}  // extern "C"
