// Resident weight matrices: upload + repack of GGUF blocks into code/scale planes,
// the inverse (download as GGUF blocks), bit-exact dequantization, and on-device
// synthetic initialisation with the GGUF quantizer rules.
#include "cai_common.cuh"
#include "gguf_blocks.cuh"

size_t cai_type_row_bytes(int type, int64_t k) {
  switch (type) {
    case CAI_TYPE_F32: return (size_t)k * 4;
    case CAI_TYPE_F16: return (size_t)k * 2;
    case CAI_TYPE_Q8_0: return (size_t)(k / CAI_QK) * CAI_Q8_0_BLOCK_BYTES;
    case CAI_TYPE_Q4_0: return (size_t)(k / CAI_QK) * CAI_Q4_0_BLOCK_BYTES;
    case CAI_TYPE_I8ROW: return (size_t)k + 4;      // codes, then the row's fp32 scale
    case CAI_TYPE_Q4_K: return (size_t)(k / 256) * 144;
    case CAI_TYPE_Q5_K: return (size_t)(k / 256) * 176;
    case CAI_TYPE_Q6_K: return (size_t)(k / 256) * 210;
  }
  return 0;
}
// K-quants that stay resident as the file's raw super-blocks (rows of K / 256 blocks, no separate scale plane)
bool cai_type_is_kquant(int type) { return type == CAI_TYPE_Q4_K || type == CAI_TYPE_Q5_K || type == CAI_TYPE_Q6_K; }
bool cai_type_supported(int type) {
  return type == CAI_TYPE_F32 || type == CAI_TYPE_F16 || type == CAI_TYPE_Q8_0 || type == CAI_TYPE_Q4_0 || type == CAI_TYPE_I8ROW ||
         cai_type_is_kquant(type);
}
size_t QWeight::row_code_bytes() const {
  switch (type) {
    case CAI_TYPE_F32: return (size_t)k * 4;
    case CAI_TYPE_F16: return (size_t)k * 2;
    case CAI_TYPE_Q8_0: return (size_t)k;
    case CAI_TYPE_I8ROW: return (size_t)k;
    case CAI_TYPE_Q4_0: return (size_t)k / 2;
    case CAI_TYPE_Q4_K: case CAI_TYPE_Q5_K: case CAI_TYPE_Q6_K: return cai_type_row_bytes(type, k);
  }
  return 0;
}
size_t QWeight::code_bytes() const { return (size_t)n * row_code_bytes(); }
size_t QWeight::scale_bytes() const {
  if (type == CAI_TYPE_Q8_0 || type == CAI_TYPE_Q4_0) return (size_t)n * (size_t)(k / CAI_QK) * 2;
  if (type == CAI_TYPE_I8ROW) return (size_t)n * 4;
  return 0;
}
size_t QWeight::scale_alloc_bytes() const {
  if (type == CAI_TYPE_Q8_0 || type == CAI_TYPE_Q4_0) return (size_t)n * (size_t)sstride * 2;
  return 0;
}

int qweight_alloc(cai_ctx* ctx, QWeight* w, int type, int64_t n, int64_t k) {
  if (!cai_type_supported(type)) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "tensor type %d is not supported (F32, F16, Q4_0, Q8_0)", type);
  if (n <= 0 || k <= 0) return cai_fail(ctx, CAI_ERR_INVALID, "weight shape %lld x %lld", (long long)n, (long long)k);
  if ((type == CAI_TYPE_Q8_0 || type == CAI_TYPE_Q4_0) && (k % CAI_QK) != 0)
    return cai_fail(ctx, CAI_ERR_INVALID, "quantized rows need a multiple of 32 columns, got %lld", (long long)k);
  if (type == CAI_TYPE_I8ROW && (k % 16) != 0)
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "int8 rows need a multiple of 16 columns, got %lld", (long long)k);
  if (cai_type_is_kquant(type) && (k % 256) != 0)
    return cai_fail(ctx, CAI_ERR_INVALID, "K-quant rows are whole super-blocks of 256 columns, got %lld", (long long)k);
  qweight_free(w);
  w->type = type; w->n = n; w->k = k; w->owns = true; w->present = false;
  // scale rows padded to 8 halves so that every row (and every 256-column tile of it) starts on a
  // 16-byte boundary, which the bulk-copy (TMA) loads of the GEMV need
  w->sstride = ((k / CAI_QK) + 7) / 8 * 8;
  size_t cb = w->code_bytes(), sb = w->scale_alloc_bytes();
  size_t free_b = 0, total_b = 0;
  cudaMemGetInfo(&free_b, &total_b);
  if (cb + sb + (64u << 20) > free_b)
    return cai_fail(ctx, CAI_ERR_OOM, "weight of %zu bytes does not fit in %zu free device bytes", cb + sb, free_b);
  // +16 bytes of slack so that 16-byte vector loads of a row tail never leave the allocation
  if (cudaMalloc(&w->codes, cb + 64) != cudaSuccess) { cudaGetLastError(); return cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc(%zu) failed", cb); }
  if (sb) {
    if (cudaMalloc((void**)&w->scales, sb + 64) != cudaSuccess) { cudaGetLastError(); cudaFree(w->codes); w->codes = nullptr; return cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc(%zu) failed", sb); }
  }
  if (type == CAI_TYPE_I8ROW) {
    if (cudaMalloc((void**)&w->rscale, (size_t)n * 4 + 64) != cudaSuccess) { cudaGetLastError(); cudaFree(w->codes); w->codes = nullptr; return cai_fail(ctx, CAI_ERR_OOM, "cudaMalloc(row scales) failed"); }
  }
  return CAI_OK;
}

void qweight_free(QWeight* w) {
  if (w->owns) {
    if (w->codes) cudaFree(w->codes);
    if (w->scales) cudaFree(w->scales);
    if (w->rscale) cudaFree(w->rscale);
    if (w->bias) cudaFree(w->bias);
  }
  w->codes = nullptr; w->scales = nullptr; w->rscale = nullptr; w->bias = nullptr; w->present = false; w->n = w->k = 0; w->type = -1;
}

QWeight qweight_rows_view(const QWeight& w, int64_t row0, int64_t nrows) {
  QWeight v = w;
  v.owns = false;
  v.n = nrows;
  v.codes = (char*)w.codes + (size_t)row0 * w.row_code_bytes();
  v.scales = w.scales ? w.scales + (size_t)row0 * (size_t)w.sstride : nullptr;
  v.rscale = w.rscale ? w.rscale + row0 : nullptr;
  v.bias = w.bias ? w.bias + row0 : nullptr;
  return v;
}

int cai_ensure_staging(cai_ctx* ctx, size_t bytes) {
  if (ctx->staging_bytes >= bytes) return CAI_OK;
  if (ctx->staging_dev) cudaFree(ctx->staging_dev);
  if (ctx->staging_pinned) cudaFreeHost(ctx->staging_pinned);
  ctx->staging_dev = nullptr; ctx->staging_pinned = nullptr; ctx->staging_bytes = 0;
  CAI_CUDA(ctx, cudaMalloc(&ctx->staging_dev, bytes));
  CAI_CUDA(ctx, cudaMallocHost(&ctx->staging_pinned, bytes));
  ctx->staging_bytes = bytes;
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// repack: staged GGUF rows -> planes. One thread per 16-bit word of a block
// (blocks are 2-byte aligned: 34 and 18 bytes).
// ---------------------------------------------------------------------------
template <int HALFWORDS /* 17 for Q8_0, 9 for Q4_0 */>
__global__ void repack_blocks_kernel(const uint16_t* __restrict__ src, int64_t nrows, int64_t blocks_per_row,
                                     uint16_t* __restrict__ codes, uint16_t* __restrict__ scales, int64_t sstride) {
  const int64_t total = nrows * blocks_per_row * HALFWORDS;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t blk = i / HALFWORDS;
    const int j = (int)(i - blk * HALFWORDS);
    const uint16_t v = src[i];
    if (j == 0) scales[(blk / blocks_per_row) * sstride + (blk % blocks_per_row)] = v;
    else codes[blk * (HALFWORDS - 1) + (j - 1)] = (HALFWORDS == 17) ? (uint16_t)(v ^ 0x8080u) : v;   // Q8_0 codes are kept biased: q + 128
  }
}
template <int HALFWORDS>
__global__ void unpack_blocks_kernel(uint16_t* __restrict__ dst, int64_t nrows, int64_t blocks_per_row,
                                     const uint16_t* __restrict__ codes, const uint16_t* __restrict__ scales, int64_t sstride) {
  const int64_t total = nrows * blocks_per_row * HALFWORDS;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t blk = i / HALFWORDS;
    const int j = (int)(i - blk * HALFWORDS);
    const uint16_t c = (j == 0) ? (uint16_t)0 : codes[blk * (HALFWORDS - 1) + (j - 1)];
    dst[i] = (j == 0) ? scales[(blk / blocks_per_row) * sstride + (blk % blocks_per_row)] : ((HALFWORDS == 17) ? (uint16_t)(c ^ 0x8080u) : c);
  }
}

// ---------------------------------------------------------------------------
// int8 rows (CAI_TYPE_I8ROW): staged host rows [K codes | fp32 scale] <-> planes (codes biased by 128, row scales)
// ---------------------------------------------------------------------------
__global__ void repack_i8rows_kernel(const uint32_t* __restrict__ src, int64_t nrows, int64_t k, uint32_t* __restrict__ codes,
                                     float* __restrict__ rscale) {
  const int64_t wpr = k / 4 + 1;                        // 32-bit words per staged row
  const int64_t total = nrows * wpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / wpr, j = i - row * wpr;
    if (j == wpr - 1) rscale[row] = __uint_as_float(src[i]);
    else codes[row * (k / 4) + j] = src[i] ^ 0x80808080u;
  }
}
__global__ void unpack_i8rows_kernel(uint32_t* __restrict__ dst, int64_t nrows, int64_t k, const uint32_t* __restrict__ codes,
                                     const float* __restrict__ rscale) {
  const int64_t wpr = k / 4 + 1;
  const int64_t total = nrows * wpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / wpr, j = i - row * wpr;
    dst[i] = (j == wpr - 1) ? __float_as_uint(rscale[row]) : (codes[row * (k / 4) + j] ^ 0x80808080u);
  }
}

// TNNetVolume.MaxAbsFinite + QuantizeInt8, scalar form (neural/neuralvolume.pas:12471-12562), one CTA per row:
// maxabs over the finite magnitudes; scale = maxabs / 127; code = Round(v * (1 / maxabs) * 127) with the products
// in that order (every intermediate bounded by 1), clamped to +-127 (which is what maps +-Inf), round-half-to-even,
// NaN -> 0; a denormal row maximum scales in double (127 / maxabs), a zero row gives zero codes and scale 0.
// Codes are stored biased by 128 like the resident Q8_0 codes. `gen` != 0: the row is not read but drawn:
// std * N(0,1) keyed by (seed, tensor, global element), the synthetic initialisation.
__device__ __forceinline__ float keyed_normal(uint64_t seed, uint64_t tensor_id, uint64_t elem);
__global__ void quantize_i8rows_kernel(const float* __restrict__ x, int64_t k, uint8_t* __restrict__ codes, float* __restrict__ rscale,
                                       int gen, uint64_t seed, uint64_t tensor_id, float std, int64_t grow0, int64_t gcol0, int64_t gcols) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  auto value = [&](int64_t c) -> float {
    if (gen) return std * keyed_normal(seed, tensor_id, (uint64_t)(grow0 + row) * (uint64_t)gcols + (uint64_t)(gcol0 + c));
    return x[row * k + c];
  };
  float m = 0.f;
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    const float a = fabsf(value(c));
    if (__float_as_uint(a) <= 0x7F7FFFFFu) m = fmaxf(m, a);            // finite magnitudes only (NaN and Inf fail the test)
  }
  m = block_max(m, red);
  if (threadIdx.x == 0) rscale[row] = m / 127.0f;
  const bool denormal = m > 0.f && __float_as_uint(m) < 0x00800000u;
  const float recip = (m > 0.f && !denormal) ? __fdiv_rn(1.0f, m) : 0.f;
  const double inv_d = denormal ? 127.0 / (double)m : 0.0;
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    const float v = value(c);
    int code = 0;
    if (m > 0.f && !(__float_as_uint(fabsf(v)) > 0x7F800000u)) {       // not NaN
      if (denormal) {
        float vc = v > m ? m : (v < -m ? -m : v);
        double sc = rint((double)vc * inv_d);
        code = (int)(sc > 127.0 ? 127.0 : (sc < -127.0 ? -127.0 : sc));
      } else {
        float sc = __fmul_rn(__fmul_rn(v, recip), 127.0f);
        sc = sc > 127.0f ? 127.0f : (sc < -127.0f ? -127.0f : sc);
        code = (int)rintf(sc);
      }
    }
    codes[row * k + c] = (uint8_t)(code + 128);
  }
}

int quantize_rows_i8_dev(cai_ctx* ctx, const float* x_dev, int64_t rows, int64_t cols, uint8_t* codes_biased_dev, float* scales_dev) {
  if (rows < 1 || rows > 0x7fffffff) return cai_fail(ctx, CAI_ERR_INVALID, "quantize: %lld rows", (long long)rows);
  quantize_i8rows_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(x_dev, cols, codes_biased_dev, scales_dev, 0, 0, 0, 0.f, 0, 0, 0);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

static inline int64_t interleave_src_row(int64_t t, int hd) {
  const int64_t h = t / hd, r = t % hd;
  return h * hd + ((r % 2 == 0) ? r / 2 : r / 2 + hd / 2);
}

int qweight_upload(cai_ctx* ctx, QWeight* w, const void* host, int64_t src_rows, int64_t src_cols,
                   int64_t row0, int64_t col0, int interleave_head_dim) {
  if (!host) return cai_fail(ctx, CAI_ERR_INVALID, "null tensor data");
  if (row0 < 0 || col0 < 0 || row0 + w->n > src_rows || col0 + w->k > src_cols)
    return cai_fail(ctx, CAI_ERR_INVALID, "slice [%lld+%lld, %lld+%lld] outside tensor %lld x %lld",
                    (long long)row0, (long long)w->n, (long long)col0, (long long)w->k, (long long)src_rows, (long long)src_cols);
  const bool quant = (w->type == CAI_TYPE_Q8_0 || w->type == CAI_TYPE_Q4_0);
  if (quant && (col0 % CAI_QK || src_cols % CAI_QK)) return cai_fail(ctx, CAI_ERR_INVALID, "column slice must align to 32-element blocks");
  if (cai_type_is_kquant(w->type) && (col0 % 256 || src_cols % 256))
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "column slice of a K-quant tensor must align to 256-element super-blocks");
  if (interleave_head_dim > 0 && (interleave_head_dim % 2 || src_rows % interleave_head_dim))
    return cai_fail(ctx, CAI_ERR_INVALID, "row interleave needs rows %% head_dim == 0 and an even head_dim");
  const bool i8row = w->type == CAI_TYPE_I8ROW;
  if (i8row && (col0 % 4)) return cai_fail(ctx, CAI_ERR_INVALID, "column slice of int8 rows must align to 4 codes");
  const size_t src_row_bytes = cai_type_row_bytes(w->type, src_cols);
  const size_t col_off = i8row ? (size_t)col0 : cai_type_row_bytes(w->type, col0);
  const size_t row_bytes = cai_type_row_bytes(w->type, w->k);
  const size_t chunk_cap = 32u << 20;
  CAI_TRY(cai_ensure_staging(ctx, chunk_cap));
  int64_t rows_per_chunk = (int64_t)(chunk_cap / row_bytes);
  if (rows_per_chunk < 1) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "row of %zu bytes exceeds the staging buffer", row_bytes);
  for (int64_t r = 0; r < w->n; r += rows_per_chunk) {
    const int64_t nr = (w->n - r < rows_per_chunk) ? (w->n - r) : rows_per_chunk;
    char* pin = (char*)ctx->staging_pinned;
    for (int64_t t = 0; t < nr; ++t) {
      int64_t g = row0 + r + t;
      if (interleave_head_dim > 0) g = interleave_src_row(g, interleave_head_dim);
      if (i8row) {      // the slice of the codes, then the scale that closes the source row
        memcpy(pin + (size_t)t * row_bytes, (const char*)host + (size_t)g * src_row_bytes + col_off, (size_t)w->k);
        memcpy(pin + (size_t)t * row_bytes + (size_t)w->k, (const char*)host + (size_t)g * src_row_bytes + (size_t)src_cols, 4);
      } else {
        memcpy(pin + (size_t)t * row_bytes, (const char*)host + (size_t)g * src_row_bytes + col_off, row_bytes);
      }
    }
    if (i8row) {
      CAI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_dev, pin, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, ctx->stream));
      const int threads = 256;
      int64_t want = (nr * (w->k / 4 + 1) + threads - 1) / threads;
      const int blocks = (int)(want > 65535 ? 65535 : (want < 1 ? 1 : want));
      repack_i8rows_kernel<<<blocks, threads, 0, ctx->stream>>>((const uint32_t*)ctx->staging_dev, nr, w->k,
          (uint32_t*)((char*)w->codes + (size_t)r * w->row_code_bytes()), w->rscale + r);
      CAI_LAUNCHED(ctx);
    } else if (!quant) {
      CAI_CUDA(ctx, cudaMemcpyAsync((char*)w->codes + (size_t)r * row_bytes, pin, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, ctx->stream));
    } else {
      CAI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_dev, pin, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, ctx->stream));
      const int64_t bpr = w->k / CAI_QK;
      const int threads = 256;
      int64_t want = (nr * bpr * 17 + threads - 1) / threads;
      const int blocks = (int)(want > 65535 ? 65535 : (want < 1 ? 1 : want));
      if (w->type == CAI_TYPE_Q8_0)
        repack_blocks_kernel<17><<<blocks, threads, 0, ctx->stream>>>((const uint16_t*)ctx->staging_dev, nr, bpr,
            (uint16_t*)((char*)w->codes + (size_t)r * w->row_code_bytes()), (uint16_t*)(w->scales + (size_t)r * w->sstride), w->sstride);
      else
        repack_blocks_kernel<9><<<blocks, threads, 0, ctx->stream>>>((const uint16_t*)ctx->staging_dev, nr, bpr,
            (uint16_t*)((char*)w->codes + (size_t)r * w->row_code_bytes()), (uint16_t*)(w->scales + (size_t)r * w->sstride), w->sstride);
      CAI_LAUNCHED(ctx);
    }
    CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the pinned buffer is reused by the next chunk
  }
  w->present = true;
  return CAI_OK;
}

int qweight_upload_quantize_i8(cai_ctx* ctx, QWeight* w, const float* host, int64_t src_rows, int64_t src_cols, int64_t row0, int64_t col0,
                               int interleave_head_dim) {
  if (!host || w->type != CAI_TYPE_I8ROW) return cai_fail(ctx, CAI_ERR_INVALID, "int8 quantizing upload: bad argument");
  if (row0 < 0 || col0 < 0 || row0 + w->n > src_rows || col0 + w->k > src_cols) return cai_fail(ctx, CAI_ERR_INVALID, "slice outside the tensor");
  if (col0 != 0 || w->k != src_cols)
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "a row's int8 scale covers the whole row: quantize before sharding columns");
  const size_t row_bytes = (size_t)w->k * 4;
  const size_t chunk_cap = 32u << 20;
  CAI_TRY(cai_ensure_staging(ctx, chunk_cap));
  const int64_t rows_per_chunk = (int64_t)(chunk_cap / row_bytes);
  if (rows_per_chunk < 1) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "row of %zu bytes exceeds the staging buffer", row_bytes);
  for (int64_t r = 0; r < w->n; r += rows_per_chunk) {
    const int64_t nr = (w->n - r < rows_per_chunk) ? (w->n - r) : rows_per_chunk;
    char* pin = (char*)ctx->staging_pinned;
    for (int64_t t = 0; t < nr; ++t) {
      int64_t g = row0 + r + t;
      if (interleave_head_dim > 0) g = interleave_src_row(g, interleave_head_dim);
      memcpy(pin + (size_t)t * row_bytes, (const char*)host + (size_t)g * (size_t)src_cols * 4, row_bytes);
    }
    CAI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_dev, pin, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, ctx->stream));
    CAI_TRY(quantize_rows_i8_dev(ctx, (const float*)ctx->staging_dev, nr, w->k, (uint8_t*)w->codes + (size_t)r * (size_t)w->k, w->rscale + r));
    CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  w->present = true;
  return CAI_OK;
}

int qweight_download_blocks(cai_ctx* ctx, const QWeight* w, void* out_host, size_t cap) {
  const size_t row_bytes = cai_type_row_bytes(w->type, w->k);
  if ((size_t)w->n * row_bytes > cap) return cai_fail(ctx, CAI_ERR_INVALID, "host buffer of %zu bytes is too small for %zu", cap, (size_t)w->n * row_bytes);
  const bool quant = (w->type == CAI_TYPE_Q8_0 || w->type == CAI_TYPE_Q4_0);
  if (w->type == CAI_TYPE_I8ROW) {
    const size_t chunk_cap = 32u << 20;
    CAI_TRY(cai_ensure_staging(ctx, chunk_cap));
    const int64_t rows_per_chunk = (int64_t)(chunk_cap / row_bytes);
    if (rows_per_chunk < 1) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "row too large for staging");
    for (int64_t r = 0; r < w->n; r += rows_per_chunk) {
      const int64_t nr = (w->n - r < rows_per_chunk) ? (w->n - r) : rows_per_chunk;
      int64_t want = (nr * (w->k / 4 + 1) + 255) / 256;
      const int blocks = (int)(want > 65535 ? 65535 : (want < 1 ? 1 : want));
      unpack_i8rows_kernel<<<blocks, 256, 0, ctx->stream>>>((uint32_t*)ctx->staging_dev, nr, w->k,
          (const uint32_t*)((const char*)w->codes + (size_t)r * w->row_code_bytes()), w->rscale + r);
      CAI_LAUNCHED(ctx);
      CAI_CUDA(ctx, cudaMemcpyAsync((char*)out_host + (size_t)r * row_bytes, ctx->staging_dev, (size_t)nr * row_bytes, cudaMemcpyDeviceToHost, ctx->stream));
      CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return CAI_OK;
  }
  if (!quant) {
    CAI_CUDA(ctx, cudaMemcpyAsync(out_host, w->codes, (size_t)w->n * row_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CAI_OK;
  }
  const size_t chunk_cap = 32u << 20;
  CAI_TRY(cai_ensure_staging(ctx, chunk_cap));
  const int64_t rows_per_chunk = (int64_t)(chunk_cap / row_bytes);
  if (rows_per_chunk < 1) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "row too large for staging");
  const int64_t bpr = w->k / CAI_QK;
  for (int64_t r = 0; r < w->n; r += rows_per_chunk) {
    const int64_t nr = (w->n - r < rows_per_chunk) ? (w->n - r) : rows_per_chunk;
    const int threads = 256;
    int64_t want = (nr * bpr * 17 + threads - 1) / threads;
    const int blocks = (int)(want > 65535 ? 65535 : (want < 1 ? 1 : want));
    if (w->type == CAI_TYPE_Q8_0)
      unpack_blocks_kernel<17><<<blocks, threads, 0, ctx->stream>>>((uint16_t*)ctx->staging_dev, nr, bpr,
          (const uint16_t*)((const char*)w->codes + (size_t)r * w->row_code_bytes()), (const uint16_t*)(w->scales + (size_t)r * w->sstride), w->sstride);
    else
      unpack_blocks_kernel<9><<<blocks, threads, 0, ctx->stream>>>((uint16_t*)ctx->staging_dev, nr, bpr,
          (const uint16_t*)((const char*)w->codes + (size_t)r * w->row_code_bytes()), (const uint16_t*)(w->scales + (size_t)r * w->sstride), w->sstride);
    CAI_LAUNCHED(ctx);
    CAI_CUDA(ctx, cudaMemcpyAsync((char*)out_host + (size_t)r * row_bytes, ctx->staging_dev, (size_t)nr * row_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// bit-exact dequantization of the resident planes: x = d * q, one fp32 multiply
// (DecodeGGMLSpan Q8_0 arm and DequantizeQ4_0 of the reference's GGUF reader).
// __half2float is exact for every half, subnormals included.
// ---------------------------------------------------------------------------
__global__ void dequant_kernel(int type, const void* __restrict__ codes, const __half* __restrict__ scales,
                               int64_t n_elems, int64_t k, int64_t sstride, float* __restrict__ out, const float* __restrict__ rscale) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += (int64_t)gridDim.x * blockDim.x) {
    float v;
    if (type == CAI_TYPE_Q8_0) {
      const float d = __half2float(scales[(i / k) * sstride + (i % k) / CAI_QK]);
      v = d * (float)((int)((const uint8_t*)codes)[i] - 128);   // resident Q8_0 codes are biased by 128
    } else if (type == CAI_TYPE_Q4_0) {
      const int64_t blk = i / CAI_QK;
      const int e = (int)(i % CAI_QK);
      const uint8_t byte = ((const uint8_t*)codes)[blk * 16 + (e & 15)];
      const int nib = (e < 16) ? (byte & 0x0F) : (byte >> 4);
      const float d = __half2float(scales[(i / k) * sstride + (i % k) / CAI_QK]);
      v = d * (float)(nib - 8);
    } else if (type == CAI_TYPE_I8ROW) {
      v = rscale[i / k] * (float)((int)((const uint8_t*)codes)[i] - 128);      // DequantizeInt8: code * row scale
    } else if (type == CAI_TYPE_F16) {
      v = __half2float(((const __half*)codes)[i]);
    } else if (type == CAI_TYPE_Q4_K || type == CAI_TYPE_Q5_K || type == CAI_TYPE_Q6_K) {
      const int bb = type == CAI_TYPE_Q4_K ? 144 : (type == CAI_TYPE_Q5_K ? 176 : 210);
      v = ggufdev::decode_element(type, (const uint8_t*)codes + (i >> 8) * bb, (int)(i & 255));    // rows are whole super-blocks
    } else {
      v = ((const float*)codes)[i];
    }
    out[i] = v;
  }
}

int qweight_dequantize_to_dev(cai_ctx* ctx, const QWeight* w, float* out_dev) {
  const int64_t n_elems = w->n * w->k;
  const int threads = 256;
  int64_t want = (n_elems + threads - 1) / threads;
  const int blocks = (int)(want > 148 * 32 ? 148 * 32 : want);
  dequant_kernel<<<blocks, threads, 0, ctx->stream>>>(w->type, w->codes, w->scales, n_elems, w->k, w->sstride, out_dev, w->rscale);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// synthetic initialisation on the device
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
// N(0,1) keyed by (seed, tensor, element): Box-Muller on two 24-bit uniforms.
__device__ __forceinline__ float keyed_normal(uint64_t seed, uint64_t tensor_id, uint64_t elem) {
  const uint64_t u = splitmix64(splitmix64(seed ^ (tensor_id * 0xD6E8FEB86659FD93ull)) + elem);
  const float u1 = (float)((u >> 40) + 1) * 5.9604644775390625e-8f;      // (0, 1]
  const float u2 = (float)(u & 0xFFFFFFu) * 5.9604644775390625e-8f;      // [0, 1)
  return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

// One warp per 32-element block; lane = element.
__global__ void synth_weight_kernel(int type, void* __restrict__ codes, __half* __restrict__ scales,
                                    int64_t n, int64_t k, int64_t sstride, uint64_t seed, uint64_t tensor_id, float std,
                                    int64_t grow0, int64_t gcol0, int64_t gcols) {
  const int lane = threadIdx.x & 31;
  const int64_t bpr = k / CAI_QK;
  const int64_t nblk = n * bpr;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < nblk; b += warps) {
    const int64_t row = b / bpr, kb = b - row * bpr;
    const int64_t col = kb * CAI_QK + lane;
    const uint64_t elem = (uint64_t)(grow0 + row) * (uint64_t)gcols + (uint64_t)(gcol0 + col);
    const float v = std * keyed_normal(seed, tensor_id, elem);
    if (type == CAI_TYPE_F32) {
      ((float*)codes)[row * k + col] = v;
    } else if (type == CAI_TYPE_F16) {
      ((__half*)codes)[row * k + col] = __float2half_rn(v);
    } else if (type == CAI_TYPE_Q8_0) {
      // the GGUF writer's Q8_0 rule: scale = absmax/127 (fp32), inverse from the
      // un-rounded scale, round half away from zero, clamp to +-127
      const float amax = warp_max(fabsf(v));
      const float scale = amax / 127.0f;
      const float inv = (scale == 0.f) ? 0.f : 1.0f / scale;
      // (explicitly un-fused: the writer rounds the product, then the sum; a fused multiply-add would round once)
      const float q = __fmul_rn(v, inv);
      int e = (q >= 0.f) ? (int)truncf(__fadd_rn(q, 0.5f)) : (int)truncf(__fadd_rn(q, -0.5f));
      e = e > 127 ? 127 : (e < -127 ? -127 : e);
      ((uint8_t*)codes)[row * k + col] = (uint8_t)(e + 128);    // biased resident form
      if (lane == 0) scales[row * sstride + kb] = __float2half_rn(scale);
    } else {  // Q4_0, ggml rule: signed value of largest magnitude (first on ties), d = max/-8
      float best = fabsf(v);
      float bestv = v;
      int besti = lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const float ov = __shfl_xor_sync(0xffffffffu, bestv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ob > best || (ob == best && oi < besti)) { best = ob; bestv = ov; besti = oi; }
      }
      const float d = bestv / -8.0f;
      const float id = (d == 0.f) ? 0.f : 1.0f / d;
      int c = (int)truncf(__fadd_rn(__fmul_rn(v, id), 8.5f));        // product rounded, then the sum, as in ggml
      c = c > 15 ? 15 : (c < 0 ? 0 : c);
      const int hi = __shfl_down_sync(0xffffffffu, c, 16);
      if (lane < 16) ((uint8_t*)codes)[b * 16 + lane] = (uint8_t)(c | (hi << 4));
      if (lane == 0) scales[row * sstride + kb] = __float2half_rn(d);
    }
  }
}

__global__ void synth_vec_kernel(float* __restrict__ v, int64_t n, uint64_t seed, uint64_t tensor_id, float std,
                                 int64_t g0, float constant) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    v[i] = (std == 0.f) ? constant : std * keyed_normal(seed, tensor_id, (uint64_t)(g0 + i));
}

int qweight_init_synthetic(cai_ctx* ctx, QWeight* w, uint64_t seed, uint64_t tensor_id, float std,
                           int64_t global_row0, int64_t global_col0, int64_t global_cols) {
  if (w->k % CAI_QK) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "synthetic init needs a multiple of 32 columns");
  if (w->type == CAI_TYPE_I8ROW) {
    quantize_i8rows_kernel<<<(unsigned)w->n, 256, 0, ctx->stream>>>(nullptr, w->k, (uint8_t*)w->codes, w->rscale, 1, seed, tensor_id, std,
                                                                   global_row0, global_col0, global_cols);
    CAI_LAUNCHED(ctx);
    w->present = true;
    return CAI_OK;
  }
  const int64_t nblk = w->n * (w->k / CAI_QK);
  const int threads = 256;
  int64_t want = (nblk * 32 + threads - 1) / threads;
  const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
  synth_weight_kernel<<<blocks, threads, 0, ctx->stream>>>(w->type, w->codes, w->scales, w->n, w->k, w->sstride, seed, tensor_id, std,
                                                           global_row0, global_col0, global_cols);
  CAI_LAUNCHED(ctx);
  w->present = true;
  return CAI_OK;
}

int vec_init_synthetic(cai_ctx* ctx, float* v, int64_t n, uint64_t seed, uint64_t tensor_id, float std,
                       int64_t global0, float constant) {
  const int threads = 256;
  int64_t want = (n + threads - 1) / threads;
  const int blocks = (int)(want > 1024 ? 1024 : want);
  synth_vec_kernel<<<blocks, threads, 0, ctx->stream>>>(v, n, seed, tensor_id, std, global0, constant);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
