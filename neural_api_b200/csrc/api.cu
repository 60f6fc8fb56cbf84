// C-ABI entry points: context, device buffers, timing, codec hook, the resident
// linear layer and the layer-granular shims. The model / session entry points
// live in model.cu.
#include "cai_common.cuh"
#include <new>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>

int cai_fail(cai_ctx* ctx, int code, const char* fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

int cai_check_device_error(cai_ctx* ctx) {
  if (ctx->err_flag && *(volatile int*)ctx->err_flag) {
    const int code = *(volatile int*)ctx->err_flag;
    *ctx->err_flag = 0;
    if (code == 2)
      return cai_fail(ctx, CAI_ERR_STATE, "a kernel refused a cache length outside [0, max_ctx): nothing was appended or attended");
    if (code == 3)
      return cai_fail(ctx, CAI_ERR_INVALID, "a kernel met a router row without a finite maximum (NaN logits): expert ids were clamped");
    if (code == 4) {
      const int site = ctx->err_flag[1], value = ctx->err_flag[2], bound = ctx->err_flag[3];
      const char* what = site == CAI_SITE_EMBED_TOKEN ? "token id in the embedding gather"
                         : site == CAI_SITE_STEP_TOKEN ? "token id in the step kernel's embedding gather"
                         : site == CAI_SITE_MOE_EXPERT ? "expert id in the mixture-of-experts grouping" : "index";
      return cai_fail(ctx, CAI_ERR_STATE, "checked build: %s: %d outside [0, %d) (the ordinary build clamps or skips it silently)", what, value, bound);
    }
    return cai_fail(ctx, CAI_ERR_CUDA, "a kernel gave up a bounded wait (device error word raised)");
  }
  return CAI_OK;
}

// Checked build only (CAI_LAUNCHED): waits for the launch just enqueued and reports what it raised, with the launch
// site. A stream that is being captured cannot be synchronized; this build does not capture (model.cu).
int cai_checked_after_launch(cai_ctx* ctx, const char* file, int line) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) { cudaGetLastError(); return CAI_OK; }
  const cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "checked build: the kernel launched at %s:%d -> %s", file, line, cudaGetErrorString(e));
  const int c = cai_check_device_error(ctx);
  if (c != CAI_OK) {
    const size_t n = strlen(ctx->err);
    snprintf(ctx->err + n, sizeof(ctx->err) - n, " [launch at %s:%d]", file, line);
  }
  return c;
}

int cai_prof_mark(cai_ctx* ctx, int family) {
  if (ctx->prof_n >= ctx->prof_cap) {
    const int ncap = ctx->prof_cap ? ctx->prof_cap * 2 : 4096;
    cudaEvent_t* ne = (cudaEvent_t*)realloc(ctx->prof_events, sizeof(cudaEvent_t) * (size_t)ncap);
    int* nf = (int*)realloc(ctx->prof_family, sizeof(int) * (size_t)ncap);
    if (!ne || !nf) return CAI_ERR_OOM;
    ctx->prof_events = ne; ctx->prof_family = nf;
    for (int i = ctx->prof_cap; i < ncap; ++i) cudaEventCreate(&ctx->prof_events[i]);
    ctx->prof_cap = ncap;
  }
  cudaEventRecord(ctx->prof_events[ctx->prof_n], ctx->stream);
  ctx->prof_family[ctx->prof_n] = family;
  ctx->prof_n++;
  return CAI_OK;
}

extern "C" {

int cai_cuda_shutdown(cai_ctx* ctx);

int cai_cuda_init(int device_id, cai_ctx** out_ctx) {
  if (!out_ctx) return CAI_ERR_INVALID;
  *out_ctx = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device_id < 0 || device_id >= count) { cudaGetLastError(); return CAI_ERR_CUDA; }
  if (cudaSetDevice(device_id) != cudaSuccess) { cudaGetLastError(); return CAI_ERR_CUDA; }
  cai_ctx* ctx = new (std::nothrow) cai_ctx();
  if (!ctx) return CAI_ERR_OOM;
  memset(ctx, 0, sizeof(*ctx));
  ctx->device = device_id;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) { delete ctx; return CAI_ERR_CUDA; }
  ctx->sm_count = prop.multiProcessorCount;
  ctx->total_mem = prop.totalGlobalMem;
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreate(&ctx->ev_begin) != cudaSuccess || cudaEventCreate(&ctx->ev_end) != cudaSuccess) {
    delete ctx;
    return CAI_ERR_CUDA;
  }
  if (cudaHostAlloc((void**)&ctx->err_flag, 4 * sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
    cudaGetLastError();
    cai_cuda_shutdown(ctx);
    return CAI_ERR_CUDA;
  }
  for (int i = 0; i < 4; ++i) ctx->err_flag[i] = 0;
  ctx->wait_limit_us = (unsigned)env_int("CAI_WAIT_LIMIT_US", 2000000);
  {
    // CAI_PDL=1 / 0 forces programmatic dependent launch on / off; unset, every session decides for its model
    // (measured on B200: +11 % tokens/s on the 0.5B model, whose step is launch-bound, -5 % on the 32B model)
    const char* e = getenv("CAI_PDL");
    ctx->pdl_mode = (e && *e) ? ((*e == '1') ? 1 : 0) : -1;
    ctx->use_pdl = ctx->pdl_mode == 1 ? 1 : 0;
  }
  *out_ctx = ctx;
  return CAI_OK;
}

int cai_cuda_is_checked_build(void) { return CAI_CHECKED_BUILD; }

int cai_cuda_set_wait_limit_us(cai_ctx* ctx, unsigned limit_us) {
  if (!ctx || limit_us < 1) return CAI_ERR_INVALID;
  ctx->wait_limit_us = limit_us;
  return CAI_OK;
}

int cai_cuda_shutdown(cai_ctx* ctx) {
  if (!ctx) return CAI_ERR_INVALID;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  comm_destroy(ctx);
  for (int i = 0; i < ctx->prof_cap; ++i) cudaEventDestroy(ctx->prof_events[i]);
  free(ctx->prof_events);
  free(ctx->prof_family);
  if (ctx->l2_flush_buf) cudaFree(ctx->l2_flush_buf);
  if (ctx->tc_xp) cudaFree(ctx->tc_xp);
  for (int i = 0; i < ctx->tc_xp_n_retired; ++i) cudaFree(ctx->tc_xp_retired[i]);
  if (ctx->err_flag) cudaFreeHost(ctx->err_flag);
  if (ctx->staging_dev) cudaFree(ctx->staging_dev);
  if (ctx->staging_pinned) cudaFreeHost(ctx->staging_pinned);
  cudaEventDestroy(ctx->ev_begin);
  cudaEventDestroy(ctx->ev_end);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return CAI_OK;
}

int cai_cuda_last_error(cai_ctx* ctx, char* buf, int buf_len) {
  if (!ctx || !buf || buf_len < 1) return CAI_ERR_INVALID;
  strncpy(buf, ctx->err, (size_t)buf_len - 1);
  buf[buf_len - 1] = 0;
  return CAI_OK;
}

int cai_cuda_device_info(cai_ctx* ctx, int* sm_count, int64_t* total_bytes) {
  if (!ctx) return CAI_ERR_INVALID;
  if (sm_count) *sm_count = ctx->sm_count;
  if (total_bytes) *total_bytes = (int64_t)ctx->total_mem;
  return CAI_OK;
}

int cai_cuda_launch_count(cai_ctx* ctx, int64_t* out_count) {
  if (!ctx || !out_count) return CAI_ERR_INVALID;
  *out_count = ctx->launches;
  return CAI_OK;
}

int cai_dev_alloc(cai_ctx* ctx, int64_t bytes, void** out_dev) {
  CAI_TRY(cai_bind(ctx));
  if (!out_dev || bytes <= 0) return cai_fail(ctx, CAI_ERR_INVALID, "cai_dev_alloc: %lld bytes", (long long)bytes);
  size_t free_b = 0, total_b = 0;
  CAI_CUDA(ctx, cudaMemGetInfo(&free_b, &total_b));
  if ((size_t)bytes > free_b) return cai_fail(ctx, CAI_ERR_OOM, "request of %lld bytes exceeds %zu free device bytes", (long long)bytes, free_b);
  if (cudaMalloc(out_dev, (size_t)bytes) != cudaSuccess) { cudaGetLastError(); return cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc(%lld) failed", (long long)bytes); }
  return CAI_OK;
}
int cai_dev_free(cai_ctx* ctx, void* dev) {
  CAI_TRY(cai_bind(ctx));
  if (dev) CAI_CUDA(ctx, cudaFree(dev));
  return CAI_OK;
}
int cai_memcpy_h2d(cai_ctx* ctx, void* dst_dev, const void* src_host, int64_t bytes) {
  CAI_TRY(cai_bind(ctx));
  if (!dst_dev || !src_host || bytes < 0) return cai_fail(ctx, CAI_ERR_INVALID, "cai_memcpy_h2d: bad argument");
  CAI_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, (size_t)bytes, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}
int cai_memcpy_d2h(cai_ctx* ctx, void* dst_host, const void* src_dev, int64_t bytes) {
  CAI_TRY(cai_bind(ctx));
  if (!dst_host || !src_dev || bytes < 0) return cai_fail(ctx, CAI_ERR_INVALID, "cai_memcpy_d2h: bad argument");
  CAI_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, (size_t)bytes, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}
int cai_dev_sync(cai_ctx* ctx) {
  CAI_TRY(cai_bind(ctx));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return cai_check_device_error(ctx);
}
int cai_timer_begin(cai_ctx* ctx) {
  CAI_TRY(cai_bind(ctx));
  CAI_CUDA(ctx, cudaEventRecord(ctx->ev_begin, ctx->stream));
  return CAI_OK;
}
int cai_timer_end(cai_ctx* ctx, float* out_ms) {
  CAI_TRY(cai_bind(ctx));
  if (!out_ms) return cai_fail(ctx, CAI_ERR_INVALID, "cai_timer_end: null output");
  CAI_CUDA(ctx, cudaEventRecord(ctx->ev_end, ctx->stream));
  CAI_CUDA(ctx, cudaEventSynchronize(ctx->ev_end));
  CAI_CUDA(ctx, cudaEventElapsedTime(out_ms, ctx->ev_begin, ctx->ev_end));
  return CAI_OK;
}
int cai_flush_l2(cai_ctx* ctx) {
  CAI_TRY(cai_bind(ctx));
  if (!ctx->l2_flush_buf) {
    ctx->l2_flush_bytes = (size_t)256 << 20;   // twice the 126 MB L2
    CAI_CUDA(ctx, cudaMalloc(&ctx->l2_flush_buf, ctx->l2_flush_bytes));
  }
  CAI_CUDA(ctx, cudaMemsetAsync(ctx->l2_flush_buf, 0, ctx->l2_flush_bytes, ctx->stream));
  return CAI_OK;
}

int cai_dequantize(cai_ctx* ctx, int type, const void* blocks_host, int64_t rows, int64_t cols, float* out_host) {
  CAI_TRY(cai_bind(ctx));
  if (!blocks_host || !out_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_dequantize: null buffer");
  if (gguf_type_needs_decode(type)) return gguf_decode_host(ctx, type, blocks_host, rows * cols, out_host);
  QWeight w;
  int st = qweight_alloc(ctx, &w, type, rows, cols);
  if (st != CAI_OK) return st;
  float* out_dev = nullptr;
  st = qweight_upload(ctx, &w, blocks_host, rows, cols, 0, 0, 0);
  if (st == CAI_OK && cudaMalloc((void**)&out_dev, (size_t)rows * cols * 4) != cudaSuccess) { cudaGetLastError(); st = cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc failed"); }
  if (st == CAI_OK) st = qweight_dequantize_to_dev(ctx, &w, out_dev);
  if (st == CAI_OK) {
    cudaError_t e = cudaMemcpyAsync(out_host, out_dev, (size_t)rows * cols * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) st = cai_fail(ctx, CAI_ERR_CUDA, "readback -> %s", cudaGetErrorString(e));
  }
  if (out_dev) cudaFree(out_dev);
  qweight_free(&w);
  return st;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// resident linear layer
// ---------------------------------------------------------------------------
struct cai_linear {
  cai_ctx* ctx;
  QWeight w;
  float* x_dev = nullptr;
  float* y_dev = nullptr;
  int cap_batch = 0;
  int path = 0;
};

static int linear_ensure_io(cai_linear* lin, int batch) {
  if (batch <= lin->cap_batch) return CAI_OK;
  cai_ctx* ctx = lin->ctx;
  if (lin->x_dev) cudaFree(lin->x_dev);
  if (lin->y_dev) cudaFree(lin->y_dev);
  lin->x_dev = lin->y_dev = nullptr; lin->cap_batch = 0;
  CAI_CUDA(ctx, cudaMalloc((void**)&lin->x_dev, (size_t)batch * lin->w.k * 4));
  CAI_CUDA(ctx, cudaMalloc((void**)&lin->y_dev, (size_t)batch * lin->w.n * 4));
  lin->cap_batch = batch;
  return CAI_OK;
}

extern "C" {

int cai_linear_create(cai_ctx* ctx, int type, const void* blocks_host, int64_t n_rows, int64_t k_cols,
                      const float* bias_host, cai_linear** out) {
  CAI_TRY(cai_bind(ctx));
  if (!out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_create: null output");
  *out = nullptr;
  if (gguf_type_needs_decode(type)) {
    // Q4_1 / Q5_x / K-quants: decoded once at load (DecodeGGMLSpan, neural/neuralgguf.pas:1471-1523), resident as F32
    if (!blocks_host || n_rows < 1 || k_cols < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_create: bad argument");
    std::vector<float> f32((size_t)n_rows * (size_t)k_cols);
    CAI_TRY(gguf_decode_host(ctx, type, blocks_host, n_rows * k_cols, f32.data()));
    return cai_linear_create(ctx, CAI_TYPE_F32, f32.data(), n_rows, k_cols, bias_host, out);
  }
  cai_linear* lin = new (std::nothrow) cai_linear();
  if (!lin) return cai_fail(ctx, CAI_ERR_OOM, "host allocation failed");
  lin->ctx = ctx;
  int st = qweight_alloc(ctx, &lin->w, type, n_rows, k_cols);
  if (st == CAI_OK) st = qweight_upload(ctx, &lin->w, blocks_host, n_rows, k_cols, 0, 0, 0);
  if (st == CAI_OK && bias_host) {
    if (cudaMalloc((void**)&lin->w.bias, (size_t)n_rows * 4) != cudaSuccess) { cudaGetLastError(); st = cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc failed"); }
    else {
      cudaError_t e = cudaMemcpyAsync(lin->w.bias, bias_host, (size_t)n_rows * 4, cudaMemcpyHostToDevice, ctx->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) st = cai_fail(ctx, CAI_ERR_CUDA, "bias upload -> %s", cudaGetErrorString(e));
    }
  }
  if (st != CAI_OK) { qweight_free(&lin->w); delete lin; return st; }
  *out = lin;
  return CAI_OK;
}

int cai_linear_create_int8(cai_ctx* ctx, const int8_t* codes_host, const float* scales_host, int64_t n_rows, int64_t k_cols,
                           const float* bias_host, cai_linear** out) {
  CAI_TRY(cai_bind(ctx));
  if (!out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_create_int8: null output");
  *out = nullptr;
  if (!codes_host || !scales_host || n_rows < 1 || k_cols < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_create_int8: bad argument");
  // the library's host row format for this type: K codes, then the row's scale
  std::vector<unsigned char> rows((size_t)n_rows * ((size_t)k_cols + 4));
  for (int64_t r = 0; r < n_rows; ++r) {
    unsigned char* dst = rows.data() + (size_t)r * ((size_t)k_cols + 4);
    memcpy(dst, codes_host + (size_t)r * (size_t)k_cols, (size_t)k_cols);
    memcpy(dst + k_cols, scales_host + r, 4);
  }
  return cai_linear_create(ctx, CAI_TYPE_I8ROW, rows.data(), n_rows, k_cols, bias_host, out);
}

int cai_quantize_int8_rows(cai_ctx* ctx, const float* w_host, int64_t rows, int64_t cols, int8_t* codes_out_host, float* scales_out_host) {
  CAI_TRY(cai_bind(ctx));
  if (!w_host || !codes_out_host || !scales_out_host || rows < 1 || cols < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_quantize_int8_rows: bad argument");
  float* x_dev = nullptr; uint8_t* c_dev = nullptr; float* s_dev = nullptr;
  const size_t n = (size_t)rows * (size_t)cols;
  int st = CAI_OK;
  if (cudaMalloc((void**)&x_dev, n * 4) != cudaSuccess || cudaMalloc((void**)&c_dev, n) != cudaSuccess || cudaMalloc((void**)&s_dev, (size_t)rows * 4) != cudaSuccess) {
    cudaGetLastError();
    st = cai_fail(ctx, CAI_ERR_OOM, "cai_quantize_int8_rows: device allocation failed");
  }
  if (st == CAI_OK && cudaMemcpyAsync(x_dev, w_host, n * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) st = cai_fail(ctx, CAI_ERR_CUDA, "upload failed");
  if (st == CAI_OK) st = quantize_rows_i8_dev(ctx, x_dev, rows, cols, c_dev, s_dev);
  if (st == CAI_OK) {
    cudaError_t e = cudaMemcpyAsync(codes_out_host, c_dev, n, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(scales_out_host, s_dev, (size_t)rows * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) st = cai_fail(ctx, CAI_ERR_CUDA, "cai_quantize_int8_rows -> %s", cudaGetErrorString(e));
    else for (size_t i = 0; i < n; ++i) codes_out_host[i] = (int8_t)((int)(unsigned char)codes_out_host[i] - 128);   // resident codes are biased
  }
  if (x_dev) cudaFree(x_dev);
  if (c_dev) cudaFree(c_dev);
  if (s_dev) cudaFree(s_dev);
  return st;
}

int cai_linear_destroy(cai_linear* lin) {
  if (!lin) return CAI_ERR_INVALID;
  cudaSetDevice(lin->ctx->device);
  cudaStreamSynchronize(lin->ctx->stream);
  if (lin->x_dev) cudaFree(lin->x_dev);
  if (lin->y_dev) cudaFree(lin->y_dev);
  qweight_free(&lin->w);
  delete lin;
  return CAI_OK;
}

int cai_linear_forward_dev(cai_linear* lin, const float* x_dev, int batch, float* y_dev, int act) {
  if (!lin) return CAI_ERR_INVALID;
  cai_ctx* ctx = lin->ctx;
  CAI_TRY(cai_bind(ctx));
  if (act < 0 || act > 3) return cai_fail(ctx, CAI_ERR_INVALID, "activation opcode %d", act);
  LinearArgs a;
  a.w = &lin->w; a.x = x_dev; a.ldx = lin->w.k; a.y = y_dev; a.ldy = lin->w.n; a.batch = batch; a.act = act; a.path = lin->path;
  return linear_launch(ctx, a);
}

int cai_linear_forward(cai_linear* lin, const float* x_host, int batch, float* y_host, int act) {
  if (!lin) return CAI_ERR_INVALID;
  cai_ctx* ctx = lin->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!x_host || !y_host || batch < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_forward: bad argument");
  CAI_TRY(linear_ensure_io(lin, batch));
  CAI_CUDA(ctx, cudaMemcpyAsync(lin->x_dev, x_host, (size_t)batch * lin->w.k * 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_TRY(cai_linear_forward_dev(lin, lin->x_dev, batch, lin->y_dev, act));
  CAI_CUDA(ctx, cudaMemcpyAsync(y_host, lin->y_dev, (size_t)batch * lin->w.n * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return cai_check_device_error(ctx);
}

int cai_linear_forward_many(cai_linear* const* lins, int count, const float* x_dev, int batch, float* y_dev, int iters) {
  if (!lins || count < 1 || !lins[0]) return CAI_ERR_INVALID;
  cai_ctx* ctx = lins[0]->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!x_dev || !y_dev || batch < 1 || iters < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_forward_many: bad argument");
  for (int it = 0; it < iters; ++it)
    for (int c = 0; c < count; ++c) {
      if (!lins[c] || lins[c]->ctx != ctx) return cai_fail(ctx, CAI_ERR_INVALID, "cai_linear_forward_many: handle %d", c);
      LinearArgs a;
      a.w = &lins[c]->w; a.x = x_dev; a.ldx = lins[c]->w.k; a.y = y_dev; a.ldy = lins[c]->w.n; a.batch = batch;
      CAI_TRY(linear_launch(ctx, a));
    }
  return CAI_OK;
}

int cai_linear_weight_bytes(cai_linear* lin, int64_t* out_bytes) {
  if (!lin || !out_bytes) return CAI_ERR_INVALID;
  *out_bytes = (int64_t)lin->w.bytes();
  return CAI_OK;
}

int cai_linear_dequantize(cai_linear* lin, float* out_host) {
  if (!lin) return CAI_ERR_INVALID;
  cai_ctx* ctx = lin->ctx;
  CAI_TRY(cai_bind(ctx));
  float* out_dev = nullptr;
  const size_t bytes = (size_t)lin->w.n * lin->w.k * 4;
  if (cudaMalloc((void**)&out_dev, bytes) != cudaSuccess) { cudaGetLastError(); return cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc(%zu) failed", bytes); }
  int st = qweight_dequantize_to_dev(ctx, &lin->w, out_dev);
  if (st == CAI_OK) {
    cudaError_t e = cudaMemcpyAsync(out_host, out_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) st = cai_fail(ctx, CAI_ERR_CUDA, "readback -> %s", cudaGetErrorString(e));
  }
  cudaFree(out_dev);
  return st;
}

int cai_linear_set_path(cai_linear* lin, int path) {
  if (!lin) return CAI_ERR_INVALID;
  if (path < 0 || path > 2) return cai_fail(lin->ctx, CAI_ERR_INVALID, "path %d", path);
  lin->path = path;
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// layer shims
// ---------------------------------------------------------------------------
int cai_rmsnorm_dev(cai_ctx* ctx, const float* x_dev, const float* gain_dev, float* y_dev, int tokens, int depth, float eps) {
  CAI_TRY(cai_bind(ctx));
  if (!x_dev || !gain_dev || !y_dev || tokens < 1 || depth < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_rmsnorm_dev: bad argument");
  return op_rmsnorm(ctx, x_dev, depth, gain_dev, y_dev, depth, tokens, depth, eps);
}

int cai_rope_dev(cai_ctx* ctx, float* x_dev, int tokens, int depth, int head_dim, int position_offset, float theta_base) {
  CAI_TRY(cai_bind(ctx));
  if (!x_dev || tokens < 1 || depth < 2 || head_dim < 2 || (head_dim % 2) || (depth % head_dim))
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_rope_dev: depth %d head_dim %d", depth, head_dim);
  float* theta = nullptr;
  CAI_CUDA(ctx, cudaMalloc((void**)&theta, (size_t)(head_dim / 2) * 4));
  int st = op_rope_theta_table(ctx, theta, head_dim, theta_base);
  if (st == CAI_OK) st = op_rope(ctx, x_dev, depth, tokens, depth, head_dim, theta, nullptr, 0, position_offset);
  cudaStreamSynchronize(ctx->stream);
  cudaFree(theta);
  return st;
}

int cai_swiglu_dev(cai_ctx* ctx, const float* x_dev, float* y_dev, int tokens, int half_depth) {
  CAI_TRY(cai_bind(ctx));
  if (!x_dev || !y_dev || tokens < 1 || half_depth < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_swiglu_dev: bad argument");
  return op_swiglu(ctx, x_dev, 2 * (int64_t)half_depth, y_dev, half_depth, tokens, half_depth);
}

int cai_topk_gate_dev(cai_ctx* ctx, const float* router_logits_dev, int tokens, int n_experts, int top_k, int renorm,
                      int32_t* expert_ids_dev, float* gates_dev) {
  CAI_TRY(cai_bind(ctx));
  if (!router_logits_dev || !expert_ids_dev || !gates_dev || tokens < 1 || n_experts < 1)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_topk_gate_dev: bad argument");
  return op_topk_gate(ctx, router_logits_dev, tokens, n_experts, top_k, renorm, expert_ids_dev, gates_dev);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// fused attention layer with its cache
// ---------------------------------------------------------------------------
struct cai_sdpa {
  cai_ctx* ctx;
  int q_heads, kv_heads, head_dim, max_ctx;
  float* k_cache = nullptr;
  float* v_cache = nullptr;
  int32_t* len_dev = nullptr;
  float* row_dev = nullptr;      // private copy of the input row
  float* partial = nullptr;
  int nsplit = 1;
  int len = 0;
  int ctx_pitch = 0;             // positions per KV head in the caches (max_ctx rounded up to 32)
  int k_blocked = 0;             // K cache block-transposed (the caches are private to the object)
  int window = 0, evict_sinks = 0, evict_window = 0;
};

extern "C" {

int cai_sdpa_create(cai_ctx* ctx, int q_heads, int kv_heads, int head_dim, int max_ctx, cai_sdpa** out) {
  CAI_TRY(cai_bind(ctx));
  if (!out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_sdpa_create: null output");
  *out = nullptr;
  if (q_heads < 1 || kv_heads < 1 || (q_heads % kv_heads) || head_dim < 2 || (head_dim % 2) || head_dim > 256 || max_ctx < 1)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_sdpa_create: heads %d/%d head_dim %d ctx %d", q_heads, kv_heads, head_dim, max_ctx);
  cai_sdpa* s = new (std::nothrow) cai_sdpa();
  if (!s) return cai_fail(ctx, CAI_ERR_OOM, "host allocation failed");
  s->ctx = ctx; s->q_heads = q_heads; s->kv_heads = kv_heads; s->head_dim = head_dim; s->max_ctx = max_ctx;
  s->ctx_pitch = (max_ctx + 31) & ~31;
  s->k_blocked = attn_k_blocked_supported(q_heads, kv_heads, head_dim) ? 1 : 0;
  const size_t cache = (size_t)kv_heads * s->ctx_pitch * head_dim * 4;
  s->nsplit = attn_nsplit(ctx, 1, kv_heads, max_ctx);
  const size_t rowf = (size_t)(q_heads + 2 * kv_heads) * head_dim;
  bool ok = cudaMalloc((void**)&s->k_cache, cache) == cudaSuccess && cudaMalloc((void**)&s->v_cache, cache) == cudaSuccess &&
            cudaMalloc((void**)&s->len_dev, 4) == cudaSuccess && cudaMalloc((void**)&s->row_dev, rowf * 4) == cudaSuccess &&
            cudaMalloc((void**)&s->partial, attn_partial_floats(1, q_heads, s->nsplit, head_dim) * 4) == cudaSuccess;
  if (!ok) { cudaGetLastError(); cai_sdpa_destroy(s); return cai_fail(ctx, CAI_ERR_OOM, "attention cache of %zu bytes does not fit", 2 * cache); }
  cudaMemsetAsync(s->len_dev, 0, 4, ctx->stream);
  *out = s;
  return CAI_OK;
}

int cai_sdpa_destroy(cai_sdpa* s) {
  if (!s) return CAI_ERR_INVALID;
  cudaSetDevice(s->ctx->device);
  cudaStreamSynchronize(s->ctx->stream);
  if (s->k_cache) cudaFree(s->k_cache);
  if (s->v_cache) cudaFree(s->v_cache);
  if (s->len_dev) cudaFree(s->len_dev);
  if (s->row_dev) cudaFree(s->row_dev);
  if (s->partial) cudaFree(s->partial);
  delete s;
  return CAI_OK;
}

static int sdpa_set_len(cai_sdpa* s, int len) {
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  s->len = len;
  CAI_CUDA(ctx, cudaMemcpyAsync(s->len_dev, &s->len, 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}
int cai_sdpa_reset(cai_sdpa* s) { return s ? sdpa_set_len(s, 0) : CAI_ERR_INVALID; }
int cai_sdpa_truncate(cai_sdpa* s, int committed_len) {
  if (!s) return CAI_ERR_INVALID;
  if (committed_len < 0 || committed_len > s->len) return cai_fail(s->ctx, CAI_ERR_INVALID, "truncate to %d outside the committed prefix of %d", committed_len, s->len);
  if (s->evict_window > 0 && s->len > s->evict_sinks + s->evict_window && committed_len != s->len)
    return cai_fail(s->ctx, CAI_ERR_STATE, "truncate after eviction has dropped rows");
  return sdpa_set_len(s, committed_len);
}
int cai_sdpa_set_window(cai_sdpa* s, int window) {
  if (!s) return CAI_ERR_INVALID;
  if (window < 0) return cai_fail(s->ctx, CAI_ERR_INVALID, "window %d", window);
  s->window = window;
  return CAI_OK;
}
int cai_sdpa_enable_eviction(cai_sdpa* s, int sink_tokens, int recent_window) {
  if (!s) return CAI_ERR_INVALID;
  if (sink_tokens < 0 || recent_window < 0 || (recent_window == 0 && sink_tokens != 0) || sink_tokens + recent_window > s->max_ctx)
    return cai_fail(s->ctx, CAI_ERR_INVALID, "eviction with %d sinks + %d recent rows in a cache of %d", sink_tokens, recent_window, s->max_ctx);
  const int cap = recent_window > 0 ? sink_tokens + recent_window : s->max_ctx;
  if (s->len > cap || (s->evict_window > 0 && s->len > s->evict_sinks + s->evict_window))
    return cai_fail(s->ctx, CAI_ERR_STATE, "the policy can change only while the cache holds no more rows than it keeps");
  s->evict_sinks = sink_tokens; s->evict_window = recent_window;
  return CAI_OK;
}
int cai_sdpa_cache_len(cai_sdpa* s, int* out_len) {
  if (!s || !out_len) return CAI_ERR_INVALID;
  *out_len = s->len;
  return CAI_OK;
}

int cai_sdpa_step_dev(cai_sdpa* s, const float* qkv_row_dev, float* out_dev) {
  if (!s) return CAI_ERR_INVALID;
  cai_ctx* ctx = s->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!qkv_row_dev || !out_dev) return cai_fail(ctx, CAI_ERR_INVALID, "cai_sdpa_step_dev: null buffer");
  if (s->len >= s->max_ctx && s->evict_window == 0) return cai_fail(ctx, CAI_ERR_STATE, "attention cache is full (%d rows)", s->max_ctx);
  const size_t rowf = (size_t)(s->q_heads + 2 * s->kv_heads) * s->head_dim;
  CAI_CUDA(ctx, cudaMemcpyAsync(s->row_dev, qkv_row_dev, rowf * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  AttnArgs a;
  a.qkv = s->row_dev; a.ld = (int64_t)rowf; a.k_cache = s->k_cache; a.v_cache = s->v_cache; a.cache_len_dev = s->len_dev;
  a.batch = 1; a.q_heads = s->q_heads; a.kv_heads = s->kv_heads; a.head_dim = s->head_dim; a.max_ctx = s->ctx_pitch; a.k_blocked = s->k_blocked;
  a.window = s->window; a.evict_sinks = s->evict_sinks; a.evict_window = s->evict_window;
  a.out = out_dev; a.ldo = (int64_t)s->q_heads * s->head_dim; a.partial = s->partial; a.nsplit = s->nsplit;
  CAI_TRY(attn_rope_append(ctx, a));
  CAI_TRY(attn_decode(ctx, a));
  s->len += 1;
  CAI_CUDA(ctx, cudaMemcpyAsync(s->len_dev, &s->len, 4, cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Mixture-of-experts expert bank, layer at a time: TNNetMoEExpertBankGateUp / TNNetMoEExpertBankDown
// (wiring neural/neuralpretrained.pas:15347-15388; device twin of the down bank neural/neural.cl:2709-2807;
// semantics tests/TestNeuralLayersExtra.pas:7773-7906)
// ---------------------------------------------------------------------------
struct cai_moe_bank {
  cai_ctx* ctx;
  int n_experts, hidden, width, type;
  std::vector<QWeight> gu, down;        // per expert: [up rows | gate rows] x hidden, hidden x width
  std::vector<int> have;                // bit 0 up, 1 gate, 2 down
  const void** d_gu_codes = nullptr; const __half** d_gu_scales = nullptr;
  const void** d_down_codes = nullptr; const __half** d_down_scales = nullptr;
  float* pair_out = nullptr; int64_t pair_cap = 0;
  bool finalized = false;
};

static int bank_ptrs(cai_ctx* ctx, const void*** dst, const std::vector<const void*>& src) {
  if (*dst) cudaFree((void*)*dst);
  *dst = nullptr;
  CAI_CUDA(ctx, cudaMalloc((void**)dst, src.size() * sizeof(void*)));
  CAI_CUDA(ctx, cudaMemcpyAsync((void*)*dst, src.data(), src.size() * sizeof(void*), cudaMemcpyHostToDevice, ctx->stream));
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

extern "C" {

int cai_moe_bank_create(cai_ctx* ctx, int n_experts, int hidden, int expert_width, int type, cai_moe_bank** out) {
  CAI_TRY(cai_bind(ctx));
  if (!out) return cai_fail(ctx, CAI_ERR_INVALID, "cai_moe_bank_create: null output");
  *out = nullptr;
  if (n_experts < 1 || hidden < 1 || expert_width < 1) return cai_fail(ctx, CAI_ERR_INVALID, "cai_moe_bank_create: bad shape");
  if (type != CAI_TYPE_F32 && type != CAI_TYPE_F16 && type != CAI_TYPE_Q8_0 && type != CAI_TYPE_Q4_0)
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "expert banks hold F32, F16, Q8_0 or Q4_0 matrices");
  cai_moe_bank* b = new (std::nothrow) cai_moe_bank();
  if (!b) return cai_fail(ctx, CAI_ERR_OOM, "host allocation failed");
  b->ctx = ctx; b->n_experts = n_experts; b->hidden = hidden; b->width = expert_width; b->type = type;
  b->gu.resize((size_t)n_experts); b->down.resize((size_t)n_experts); b->have.assign((size_t)n_experts, 0);
  *out = b;
  return CAI_OK;
}

int cai_moe_bank_destroy(cai_moe_bank* b) {
  if (!b) return CAI_ERR_INVALID;
  cai_bind(b->ctx);
  for (auto& w : b->gu) qweight_free(&w);
  for (auto& w : b->down) qweight_free(&w);
  if (b->d_gu_codes) cudaFree((void*)b->d_gu_codes);
  if (b->d_gu_scales) cudaFree((void*)b->d_gu_scales);
  if (b->d_down_codes) cudaFree((void*)b->d_down_codes);
  if (b->d_down_scales) cudaFree((void*)b->d_down_scales);
  if (b->pair_out) cudaFree(b->pair_out);
  delete b;
  return CAI_OK;
}

int cai_moe_bank_upload(cai_moe_bank* b, int expert, int which, const void* blocks_host) {
  if (!b) return CAI_ERR_INVALID;
  cai_ctx* ctx = b->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!blocks_host || expert < 0 || expert >= b->n_experts || which < 0 || which > 2)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_moe_bank_upload: bad argument");
  b->finalized = false;
  if (which == 2) {
    QWeight* w = &b->down[(size_t)expert];
    if (!w->codes) CAI_TRY(qweight_alloc(ctx, w, b->type, b->hidden, b->width));
    CAI_TRY(qweight_upload(ctx, w, blocks_host, b->hidden, b->width, 0, 0, 0));
  } else {
    QWeight* w = &b->gu[(size_t)expert];
    if (!w->codes) CAI_TRY(qweight_alloc(ctx, w, b->type, 2 * (int64_t)b->width, b->hidden));
    QWeight view = qweight_rows_view(*w, which == 0 ? 0 : b->width, b->width);      // up rows first, gate rows second
    CAI_TRY(qweight_upload(ctx, &view, blocks_host, b->width, b->hidden, 0, 0, 0));
    w->present = true;
  }
  b->have[(size_t)expert] |= 1 << which;
  return CAI_OK;
}

int cai_moe_bank_finalize(cai_moe_bank* b) {
  if (!b) return CAI_ERR_INVALID;
  cai_ctx* ctx = b->ctx;
  CAI_TRY(cai_bind(ctx));
  std::vector<const void*> gc, gs, dc, ds;
  for (int e = 0; e < b->n_experts; ++e) {
    if (b->have[(size_t)e] != 7) return cai_fail(ctx, CAI_ERR_STATE, "expert %d is missing matrices (have mask 0x%x)", e, b->have[(size_t)e]);
    gc.push_back(b->gu[(size_t)e].codes); gs.push_back(b->gu[(size_t)e].scales);
    dc.push_back(b->down[(size_t)e].codes); ds.push_back(b->down[(size_t)e].scales);
  }
  CAI_TRY(bank_ptrs(ctx, &b->d_gu_codes, gc));
  CAI_TRY(bank_ptrs(ctx, (const void***)&b->d_gu_scales, gs));
  CAI_TRY(bank_ptrs(ctx, &b->d_down_codes, dc));
  CAI_TRY(bank_ptrs(ctx, (const void***)&b->d_down_scales, ds));
  b->finalized = true;
  return CAI_OK;
}

int cai_moe_gate_up_dev(cai_moe_bank* b, const float* x_dev, const int32_t* slot_expert_dev, int tokens, int top_k, float* hidden_out_dev) {
  if (!b) return CAI_ERR_INVALID;
  cai_ctx* ctx = b->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!b->finalized) return cai_fail(ctx, CAI_ERR_STATE, "cai_moe_bank_finalize first");
  if (!x_dev || !slot_expert_dev || !hidden_out_dev || tokens < 1 || top_k < 1 || top_k > b->n_experts)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_moe_gate_up_dev: bad argument");
  LinearArgs a; a.w = &b->gu[0]; a.x = x_dev; a.ldx = b->hidden; a.y = hidden_out_dev; a.ldy = b->width; a.batch = tokens * top_k;
  a.epilogue = EPI_SWIGLU; a.bank_codes_dev = b->d_gu_codes; a.bank_scales_dev = b->d_gu_scales; a.bank_count = b->n_experts;
  a.expert_ids_dev = slot_expert_dev; a.x_row_div = top_k;
  return linear_launch(ctx, a);
}

int cai_moe_down_dev(cai_moe_bank* b, const float* hidden_dev, const int32_t* slot_expert_dev, const float* slot_gate_dev, int tokens, int top_k,
                     float* out_dev) {
  if (!b) return CAI_ERR_INVALID;
  cai_ctx* ctx = b->ctx;
  CAI_TRY(cai_bind(ctx));
  if (!b->finalized) return cai_fail(ctx, CAI_ERR_STATE, "cai_moe_bank_finalize first");
  if (!hidden_dev || !slot_expert_dev || !slot_gate_dev || !out_dev || tokens < 1 || top_k < 1 || top_k > b->n_experts)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_moe_down_dev: bad argument");
  const int64_t pairs = (int64_t)tokens * top_k;
  if (pairs > b->pair_cap) {
    if (b->pair_out) cudaFree(b->pair_out);
    b->pair_out = nullptr; b->pair_cap = 0;
    CAI_CUDA(ctx, cudaMalloc((void**)&b->pair_out, (size_t)pairs * b->hidden * 4));
    b->pair_cap = pairs;
  }
  LinearArgs a; a.w = &b->down[0]; a.x = hidden_dev; a.ldx = b->width; a.y = b->pair_out; a.ldy = b->hidden; a.batch = (int)pairs;
  a.bank_codes_dev = b->d_down_codes; a.bank_scales_dev = b->d_down_scales; a.bank_count = b->n_experts; a.expert_ids_dev = slot_expert_dev; a.x_row_div = 1;
  CAI_TRY(linear_launch(ctx, a));
  // out[t] = sum over the token's slots, in slot order, of gate * down_e(hidden)   (acc = mad(g, d, acc), neural.cl:2749)
  CAI_CUDA(ctx, cudaMemsetAsync(out_dev, 0, (size_t)tokens * b->hidden * 4, ctx->stream));
  return op_moe_combine(ctx, out_dev, b->hidden, b->pair_out, b->hidden, slot_gate_dev, tokens, top_k, b->hidden);
}

}  // extern "C"
