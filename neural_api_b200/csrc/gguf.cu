// GGUF on the C side: the container reader (header, metadata, tensor table), the block decoders of every ggml type
// the reference's reader decodes (run on the device, raw file bytes in, fp32 out) and the model loader that maps a
// llama / qwen2 file onto cai_model_upload_tensor.
//   reader        TNNetGGUFReader.ParseFile            neural/neuralgguf.pas:1072-1220
//   metadata      ReadMetaValue, GetMetaInt/Float/...  neural/neuralgguf.pas:984-1069, 1263-1344
//   decoders      DequantizeQ4K ... DequantizeQ5_1      neural/neuralgguf.pas:448-945
//   model loader  BuildLlamaFromGGUFEx, BuildFromGGUFEx neural/neuralpretrained.pas:17484-17876
#include "cai_common.cuh"
#include "gguf_blocks.cuh"

#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

// ---------------------------------------------------------------------------
// block geometry (GGMLByteSize / GGMLBlockElems, neural/neuralgguf.pas:375-423)
// ---------------------------------------------------------------------------
static bool ggml_block(int type, int* bytes, int* elems) {
  switch (type) {
    case 0: *bytes = 4; *elems = 1; return true;
    case 1: *bytes = 2; *elems = 1; return true;
    case 2: *bytes = 18; *elems = 32; return true;
    case 3: *bytes = 20; *elems = 32; return true;
    case 6: *bytes = 22; *elems = 32; return true;
    case 7: *bytes = 24; *elems = 32; return true;
    case 8: *bytes = 34; *elems = 32; return true;
    case 10: *bytes = 84; *elems = 256; return true;
    case 11: *bytes = 110; *elems = 256; return true;
    case 12: *bytes = 144; *elems = 256; return true;
    case 13: *bytes = 176; *elems = 256; return true;
    case 14: *bytes = 210; *elems = 256; return true;
    default: return false;
  }
}

static const char* ggml_type_name(int t) {
  switch (t) {
    case 0: return "F32"; case 1: return "F16"; case 2: return "Q4_0"; case 3: return "Q4_1"; case 6: return "Q5_0";
    case 7: return "Q5_1"; case 8: return "Q8_0"; case 9: return "Q8_1"; case 10: return "Q2_K"; case 11: return "Q3_K";
    case 12: return "Q4_K"; case 13: return "Q5_K"; case 14: return "Q6_K"; case 15: return "Q8_K"; case 24: return "I8";
    case 25: return "I16"; case 26: return "I32"; case 27: return "I64"; case 28: return "F64"; case 30: return "BF16";
    default: return "GGML_TYPE_?";
  }
}

namespace {
using namespace ggufdev;

__global__ void gguf_decode_kernel(int type, int block_bytes, int block_elems, const uint8_t* __restrict__ raw, int64_t n_elems,
                                   float* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_elems; e += stride) {
    if (type == 0) {
      const uint8_t* p = raw + e * 4;
      out[e] = __uint_as_float(p[0] | (p[1] << 8) | (p[2] << 16) | ((unsigned)p[3] << 24));
    } else if (type == 1) {
      out[e] = f16_at(raw + e * 2);
    } else {
      const int64_t b = e / block_elems;
      out[e] = decode_element(type, raw + b * block_bytes, (int)(e - b * block_elems));
    }
  }
}

}  // namespace

// Raw tensor bytes on the host -> fp32 on the host, decoded on the device in bounded chunks (the staged chunks of
// ReadGGMLSpanInto, neural/neuralgguf.pas:1525-1569).
int gguf_decode_host(cai_ctx* ctx, int type, const void* raw_host, int64_t n_elems, float* out_host) {
  int bb, be;
  if (!ggml_block(type, &bb, &be)) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "gguf: type %d (%s) has no decoder", type, ggml_type_name(type));
  if (n_elems < 0 || n_elems % be) return cai_fail(ctx, CAI_ERR_INVALID, "gguf: %lld elements is not a whole number of %s blocks", (long long)n_elems, ggml_type_name(type));
  const int64_t chunk_elems = ((int64_t)8 << 20) / be * be;            // 8 Mi elements per chunk
  const int64_t ce = n_elems < chunk_elems ? n_elems : chunk_elems;
  if (ce == 0) return CAI_OK;
  uint8_t* raw_dev = nullptr; float* out_dev = nullptr;
  if (cudaMalloc((void**)&raw_dev, (size_t)(ce / be) * bb) != cudaSuccess || cudaMalloc((void**)&out_dev, (size_t)ce * 4) != cudaSuccess) {
    cudaGetLastError();
    if (raw_dev) cudaFree(raw_dev);
    return cai_fail(ctx, CAI_ERR_OOM, "gguf: device staging allocation failed");
  }
  int st = CAI_OK;
  for (int64_t e0 = 0; e0 < n_elems && st == CAI_OK; e0 += ce) {
    const int64_t n = (n_elems - e0) < ce ? (n_elems - e0) : ce;
    const size_t bytes = (size_t)(n / be) * bb;
    cudaError_t e = cudaMemcpyAsync(raw_dev, (const uint8_t*)raw_host + (size_t)(e0 / be) * bb, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
      const int threads = 256;
      const int64_t want = (n + threads - 1) / threads;
      const int blocks = (int)(want < (int64_t)ctx->sm_count * 8 ? want : (int64_t)ctx->sm_count * 8);
      gguf_decode_kernel<<<blocks, threads, 0, ctx->stream>>>(type, bb, be, raw_dev, n, out_dev);
      ctx->launches++;
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(out_host + e0, out_dev, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) st = cai_fail(ctx, CAI_ERR_CUDA, "gguf decode -> %s", cudaGetErrorString(e));
  }
  cudaFree(raw_dev);
  cudaFree(out_dev);
  return st;
}

// ---------------------------------------------------------------------------
// container reader (host)
// ---------------------------------------------------------------------------
struct GGUFMeta {
  int type = 0, elem_type = 0;
  int64_t i = 0; double f = 0; std::string s;
  std::vector<int64_t> arr_i; std::vector<double> arr_f; std::vector<std::string> arr_s;
};
struct GGUFTensor {
  std::string name;
  int type = 0, ndims = 0;
  int64_t shape[8] = {0};        // served order: contiguous axis LAST (the stored dims reversed, :1157-1162)
  int64_t begin = 0, end = 0;    // byte range relative to the data section
  int64_t n_elems = 0;
};
struct cai_gguf {
  std::string path;
  FILE* f = nullptr;
  int64_t file_size = 0, data_start = 0, data_size = 0;
  int version = 0, alignment = 32;
  std::vector<std::pair<std::string, GGUFMeta>> meta;
  std::map<std::string, int> meta_index;
  std::vector<GGUFTensor> tensors;
  std::map<std::string, int> tensor_index;
  std::string err;
};

namespace {

struct Parser {
  cai_gguf* g;
  bool failed = false;
  bool fail(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g->err = std::string(buf) + ": " + g->path;
    failed = true;
    return false;
  }
  bool read(void* dst, size_t n) {
    if (fread(dst, 1, n, g->f) != n) return fail("gguf: read past the end of file at offset %lld", (long long)ftello(g->f));
    return true;
  }
  template <typename T> bool get(T* v) { return read(v, sizeof(T)); }
  bool str(std::string* out) {
    uint64_t len;
    if (!get(&len)) return false;
    const int64_t pos = ftello(g->f);
    if (len > (uint64_t)(g->file_size - pos)) return fail("gguf: string length %llu at offset %lld runs past the end of file", (unsigned long long)len, (long long)(pos - 8));
    out->resize((size_t)len);
    return len == 0 || read(&(*out)[0], (size_t)len);
  }
  bool scalar(int t, const std::string& key, int64_t* iv, double* fv, std::string* sv) {
    *iv = 0; *fv = 0; sv->clear();
    switch (t) {
      case 0: { uint8_t v; if (!get(&v)) return false; *iv = v; break; }
      case 1: { int8_t v; if (!get(&v)) return false; *iv = v; break; }
      case 2: { uint16_t v; if (!get(&v)) return false; *iv = v; break; }
      case 3: { int16_t v; if (!get(&v)) return false; *iv = v; break; }
      case 4: { uint32_t v; if (!get(&v)) return false; *iv = v; break; }
      case 5: { int32_t v; if (!get(&v)) return false; *iv = v; break; }
      case 10: { uint64_t v; if (!get(&v)) return false; *iv = (int64_t)v; break; }
      case 11: { int64_t v; if (!get(&v)) return false; *iv = v; break; }
      case 6: { float v; if (!get(&v)) return false; *fv = v; return true; }
      case 12: { double v; if (!get(&v)) return false; *fv = v; return true; }
      case 7: { uint8_t v; if (!get(&v)) return false; *iv = v; break; }
      case 8: if (!str(sv)) return false; break;
      default: return fail("gguf: metadata key \"%s\" has unsupported value type %d", key.c_str(), t);
    }
    *fv = (double)*iv;
    return true;
  }
  bool parse() {
    if (g->file_size < 24) return fail("gguf: file too small (%lld bytes; need at least the 24-byte header)", (long long)g->file_size);
    uint32_t magic, u32;
    uint64_t n_tensors, n_kv, u64;
    if (!get(&magic)) return false;
    if (magic != 0x46554747u) return fail("gguf: bad magic 0x%08X (expected \"GGUF\")", magic);
    if (!get(&u32)) return false;
    g->version = (int)u32;
    if (g->version != 2 && g->version != 3) return fail("gguf: unsupported version %d (supported: 2, 3)", g->version);
    if (!get(&n_tensors) || !get(&n_kv)) return false;
    if (n_tensors > 0x7FFFFFFFull || n_kv > 0x7FFFFFFFull)
      return fail("gguf: implausible header counts (%llu tensors, %llu KV pairs)", (unsigned long long)n_tensors, (unsigned long long)n_kv);
    for (uint64_t i = 0; i < n_kv; ++i) {
      std::string key;
      if (!str(&key)) return false;
      if (key.empty()) return fail("gguf: empty metadata key (pair %llu)", (unsigned long long)i);
      if (g->meta_index.count(key)) return fail("gguf: duplicate metadata key \"%s\"", key.c_str());
      GGUFMeta m;
      if (!get(&u32)) return false;
      m.type = (int)u32;
      if (m.type == 9) {
        if (!get(&u32)) return false;
        m.elem_type = (int)u32;
        if (m.elem_type == 9) return fail("gguf: metadata key \"%s\" is a nested array (not supported)", key.c_str());
        if (!get(&u64)) return false;
        if (u64 > 0x7FFFFFFFull) return fail("gguf: metadata array \"%s\" is too large (%llu elements)", key.c_str(), (unsigned long long)u64);
        for (uint64_t k = 0; k < u64; ++k) {
          int64_t iv; double fv; std::string sv;
          if (!scalar(m.elem_type, key, &iv, &fv, &sv)) return false;
          if (m.elem_type == 8) m.arr_s.push_back(sv);
          else { m.arr_i.push_back(iv); m.arr_f.push_back(fv); }
        }
      } else if (!scalar(m.type, key, &m.i, &m.f, &m.s)) {
        return false;
      }
      g->meta_index[key] = (int)g->meta.size();
      g->meta.emplace_back(key, std::move(m));
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
      GGUFTensor t;
      if (!str(&t.name)) return false;
      if (t.name.empty()) return fail("gguf: empty tensor name (tensor %llu)", (unsigned long long)i);
      if (g->tensor_index.count(t.name)) return fail("gguf: duplicate tensor name \"%s\"", t.name.c_str());
      if (!get(&u32)) return false;
      t.ndims = (int)u32;
      if (t.ndims < 1 || t.ndims > 8) return fail("gguf: tensor \"%s\" has implausible n_dims %d", t.name.c_str(), t.ndims);
      int64_t dims[8];
      t.n_elems = 1;
      for (int j = 0; j < t.ndims; ++j) {
        if (!get(&u64)) return false;
        if (u64 == 0 || u64 > 0x7FFFFFFFull) return fail("gguf: tensor \"%s\" has implausible dimension %llu", t.name.c_str(), (unsigned long long)u64);
        dims[j] = (int64_t)u64;
        t.n_elems *= dims[j];
      }
      for (int j = 0; j < t.ndims; ++j) t.shape[j] = dims[t.ndims - 1 - j];
      if (!get(&u32)) return false;
      t.type = (int)u32;
      const bool legacy = t.type == 8 || t.type == 2 || t.type == 3 || t.type == 6 || t.type == 7;
      const bool kq = t.type >= 10 && t.type <= 14;
      if (legacy && dims[0] % 32)
        return fail("gguf: tensor \"%s\" is %s but its contiguous dimension %lld is not a multiple of the block size 32", t.name.c_str(),
                    ggml_type_name(t.type), (long long)dims[0]);
      if (kq && dims[0] % 256)
        return fail("gguf: tensor \"%s\" is %s but its contiguous dimension %lld is not a multiple of the k-quant super-block size 256",
                    t.name.c_str(), ggml_type_name(t.type), (long long)dims[0]);
      if (!get(&u64)) return false;
      t.begin = (int64_t)u64;
      int bb, be;
      // a type without a decoder keeps end == begin: the table stays inspectable, loading it fails (:1196-1200)
      t.end = t.begin + (ggml_block(t.type, &bb, &be) ? (t.n_elems / be) * bb : 0);
      g->tensor_index[t.name] = (int)g->tensors.size();
      g->tensors.push_back(t);
    }
    int64_t align = 32;
    auto it = g->meta_index.find("general.alignment");
    if (it != g->meta_index.end()) {
      const GGUFMeta& m = g->meta[(size_t)it->second].second;
      const bool is_int = m.type <= 5 || m.type == 7 || m.type == 10 || m.type == 11;
      if (!is_int) return fail("gguf: metadata key \"general.alignment\" (type %d) is not an integer", m.type);
      align = m.i;
    }
    if (align < 1 || (align & (align - 1)) || align > 0x7FFFFFFF) return fail("gguf: general.alignment %lld is not a positive power of two", (long long)align);
    g->alignment = (int)align;
    const int64_t pos = ftello(g->f);
    g->data_start = (pos + align - 1) / align * align;
    if (g->data_start > g->file_size) return fail("gguf: header ends at %lld past the end of the %lld-byte file", (long long)g->data_start, (long long)g->file_size);
    g->data_size = g->file_size - g->data_start;
    for (const GGUFTensor& t : g->tensors)
      if (t.begin < 0 || t.end > g->data_size)
        return fail("gguf: tensor \"%s\" data [%lld, %lld) falls outside the data section (size %lld)", t.name.c_str(), (long long)t.begin,
                    (long long)t.end, (long long)g->data_size);
    return true;
  }
};

void copy_str(const std::string& s, char* buf, int cap) {
  if (!buf || cap <= 0) return;
  const size_t n = s.size() < (size_t)cap - 1 ? s.size() : (size_t)cap - 1;
  memcpy(buf, s.data(), n);
  buf[n] = 0;
}

const GGUFMeta* find_meta(const cai_gguf* g, const char* key) {
  auto it = g->meta_index.find(key);
  return it == g->meta_index.end() ? nullptr : &g->meta[(size_t)it->second].second;
}

bool meta_is_int(int t) { return t <= 5 || t == 7 || t == 10 || t == 11; }

}  // namespace

extern "C" {

int cai_gguf_open(const char* path, cai_gguf** out, char* err_buf, int err_len) {
  if (err_buf && err_len > 0) err_buf[0] = 0;
  if (!path || !out) return CAI_ERR_INVALID;
  *out = nullptr;
  cai_gguf* g = new (std::nothrow) cai_gguf();
  if (!g) return CAI_ERR_OOM;
  g->path = path;
  g->f = fopen(path, "rb");
  if (!g->f) {
    copy_str(std::string("gguf: cannot open ") + path + ": " + strerror(errno), err_buf, err_len);
    delete g;
    return CAI_ERR_INVALID;
  }
  fseeko(g->f, 0, SEEK_END);
  g->file_size = ftello(g->f);
  fseeko(g->f, 0, SEEK_SET);
  Parser p{g};
  if (!p.parse()) {
    copy_str(g->err, err_buf, err_len);
    fclose(g->f);
    delete g;
    return CAI_ERR_INVALID;
  }
  *out = g;
  return CAI_OK;
}

int cai_gguf_close(cai_gguf* g) {
  if (!g) return CAI_ERR_INVALID;
  if (g->f) fclose(g->f);
  delete g;
  return CAI_OK;
}

int cai_gguf_last_error(cai_gguf* g, char* buf, int buf_len) {
  if (!g) return CAI_ERR_INVALID;
  copy_str(g->err, buf, buf_len);
  return CAI_OK;
}

int cai_gguf_info(cai_gguf* g, int* version, int* alignment, int64_t* n_meta, int64_t* n_tensors, int64_t* data_start) {
  if (!g) return CAI_ERR_INVALID;
  if (version) *version = g->version;
  if (alignment) *alignment = g->alignment;
  if (n_meta) *n_meta = (int64_t)g->meta.size();
  if (n_tensors) *n_tensors = (int64_t)g->tensors.size();
  if (data_start) *data_start = g->data_start;
  return CAI_OK;
}

int cai_gguf_meta_key(cai_gguf* g, int64_t index, char* key_buf, int key_cap, int* value_type) {
  if (!g) return CAI_ERR_INVALID;
  if (index < 0 || index >= (int64_t)g->meta.size()) { g->err = "gguf: metadata index out of range"; return CAI_ERR_INVALID; }
  copy_str(g->meta[(size_t)index].first, key_buf, key_cap);
  if (value_type) *value_type = g->meta[(size_t)index].second.type;
  return CAI_OK;
}

// found = 0 leaves *out untouched (the caller's default stands); a key of the wrong type is an error, as in the reference.
int cai_gguf_meta_int(cai_gguf* g, const char* key, int64_t* out, int* found) {
  if (!g || !key) return CAI_ERR_INVALID;
  const GGUFMeta* m = find_meta(g, key);
  if (found) *found = m != nullptr;
  if (!m) return CAI_OK;
  if (!meta_is_int(m->type)) { g->err = std::string("gguf: metadata key \"") + key + "\" is not an integer: " + g->path; return CAI_ERR_INVALID; }
  if (out) *out = m->i;
  return CAI_OK;
}

int cai_gguf_meta_float(cai_gguf* g, const char* key, double* out, int* found) {
  if (!g || !key) return CAI_ERR_INVALID;
  const GGUFMeta* m = find_meta(g, key);
  if (found) *found = m != nullptr;
  if (!m) return CAI_OK;
  const bool ok = m->type == 6 || m->type == 12 || (meta_is_int(m->type) && m->type != 7);
  if (!ok) { g->err = std::string("gguf: metadata key \"") + key + "\" is not a number: " + g->path; return CAI_ERR_INVALID; }
  if (out) *out = m->f;
  return CAI_OK;
}

int cai_gguf_meta_string(cai_gguf* g, const char* key, char* buf, int cap, int* found) {
  if (!g || !key) return CAI_ERR_INVALID;
  const GGUFMeta* m = find_meta(g, key);
  if (found) *found = m != nullptr;
  if (!m) return CAI_OK;
  if (m->type != 8) { g->err = std::string("gguf: metadata key \"") + key + "\" is not a string: " + g->path; return CAI_ERR_INVALID; }
  copy_str(m->s, buf, cap);
  return CAI_OK;
}

int cai_gguf_meta_array_count(cai_gguf* g, const char* key, int64_t* out_count) {
  if (!g || !key || !out_count) return CAI_ERR_INVALID;
  const GGUFMeta* m = find_meta(g, key);
  *out_count = 0;
  if (!m) return CAI_OK;
  if (m->type != 9) { g->err = std::string("gguf: metadata key \"") + key + "\" is not an array: " + g->path; return CAI_ERR_INVALID; }
  *out_count = (int64_t)(m->elem_type == 8 ? m->arr_s.size() : m->arr_i.size());
  return CAI_OK;
}

int cai_gguf_tensor_info(cai_gguf* g, int64_t index, char* name_buf, int name_cap, int* type, int* ndims, int64_t* shape8,
                         int64_t* data_begin, int64_t* data_bytes) {
  if (!g) return CAI_ERR_INVALID;
  if (index < 0 || index >= (int64_t)g->tensors.size()) { g->err = "gguf: tensor index out of range"; return CAI_ERR_INVALID; }
  const GGUFTensor& t = g->tensors[(size_t)index];
  copy_str(t.name, name_buf, name_cap);
  if (type) *type = t.type;
  if (ndims) *ndims = t.ndims;
  if (shape8) for (int j = 0; j < 8; ++j) shape8[j] = j < t.ndims ? t.shape[j] : 0;
  if (data_begin) *data_begin = t.begin;
  if (data_bytes) *data_bytes = t.end - t.begin;
  return CAI_OK;
}

int cai_gguf_find_tensor(cai_gguf* g, const char* name, int64_t* out_index) {
  if (!g || !name || !out_index) return CAI_ERR_INVALID;
  auto it = g->tensor_index.find(name);
  *out_index = it == g->tensor_index.end() ? -1 : it->second;
  return CAI_OK;
}

int cai_gguf_read_raw(cai_gguf* g, int64_t index, void* out_host, int64_t cap_bytes) {
  if (!g || !out_host) return CAI_ERR_INVALID;
  if (index < 0 || index >= (int64_t)g->tensors.size()) { g->err = "gguf: tensor index out of range"; return CAI_ERR_INVALID; }
  const GGUFTensor& t = g->tensors[(size_t)index];
  const int64_t n = t.end - t.begin;
  if (n > cap_bytes) { g->err = "gguf: output buffer too small for tensor \"" + t.name + "\""; return CAI_ERR_INVALID; }
  if (fseeko(g->f, g->data_start + t.begin, SEEK_SET) != 0 || (n > 0 && fread(out_host, 1, (size_t)n, g->f) != (size_t)n)) {
    g->err = "gguf: short read of tensor \"" + t.name + "\": " + g->path;
    return CAI_ERR_INVALID;
  }
  return CAI_OK;
}

int cai_gguf_decode(cai_ctx* ctx, int type, const void* raw_host, int64_t n_elems, float* out_host) {
  CAI_TRY(cai_bind(ctx));
  if (!raw_host || !out_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_gguf_decode: null buffer");
  return gguf_decode_host(ctx, type, raw_host, n_elems, out_host);
}

int cai_gguf_load_tensor(cai_ctx* ctx, cai_gguf* g, int64_t index, float* out_host, int64_t cap_elems) {
  CAI_TRY(cai_bind(ctx));
  if (!g || !out_host) return cai_fail(ctx, CAI_ERR_INVALID, "cai_gguf_load_tensor: null argument");
  if (index < 0 || index >= (int64_t)g->tensors.size()) return cai_fail(ctx, CAI_ERR_INVALID, "gguf: tensor index out of range");
  const GGUFTensor& t = g->tensors[(size_t)index];
  int bb, be;
  if (!ggml_block(t.type, &bb, &be))
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "gguf: tensor \"%s\" has unsupported type %s", t.name.c_str(), ggml_type_name(t.type));
  if (t.n_elems > cap_elems) return cai_fail(ctx, CAI_ERR_INVALID, "gguf: output buffer too small for tensor \"%s\"", t.name.c_str());
  std::vector<uint8_t> raw((size_t)(t.end - t.begin));
  if (cai_gguf_read_raw(g, index, raw.data(), (int64_t)raw.size()) != CAI_OK) return cai_fail(ctx, CAI_ERR_INVALID, "%s", g->err.c_str());
  return gguf_decode_host(ctx, t.type, raw.data(), t.n_elems, out_host);
}

// ---------------------------------------------------------------------------
// model loader
// ---------------------------------------------------------------------------
static bool map_name(const std::string& n, bool qwen2, std::string* hf) {
  if (n == "token_embd.weight") { *hf = "model.embed_tokens.weight"; return true; }
  if (n == "output_norm.weight") { *hf = "model.norm.weight"; return true; }
  if (n == "output.weight") { *hf = "lm_head.weight"; return true; }
  if (n.compare(0, 4, "blk.") != 0) return false;
  const size_t dot = n.find('.', 4);
  if (dot == std::string::npos) return false;
  const std::string layer = n.substr(4, dot - 4), rest = n.substr(dot + 1);
  static const char* const table[][2] = {
      {"attn_norm.weight", "input_layernorm.weight"}, {"attn_q.weight", "self_attn.q_proj.weight"},
      {"attn_k.weight", "self_attn.k_proj.weight"},   {"attn_v.weight", "self_attn.v_proj.weight"},
      {"attn_output.weight", "self_attn.o_proj.weight"}, {"ffn_norm.weight", "post_attention_layernorm.weight"},
      {"ffn_gate.weight", "mlp.gate_proj.weight"},    {"ffn_up.weight", "mlp.up_proj.weight"},
      {"ffn_down.weight", "mlp.down_proj.weight"}};
  for (auto& row : table)
    if (rest == row[0]) { *hf = "model.layers." + layer + "." + row[1]; return true; }
  if (qwen2) {
    static const char* const bias[][2] = {{"attn_q.bias", "self_attn.q_proj.bias"}, {"attn_k.bias", "self_attn.k_proj.bias"},
                                          {"attn_v.bias", "self_attn.v_proj.bias"}};
    for (auto& row : bias)
      if (rest == row[0]) { *hf = "model.layers." + layer + "." + row[1]; return true; }
  }
  return false;
}

int cai_gguf_llama_config(cai_gguf* g, cai_llama_config* cfg, int64_t* max_positions) {
  if (!g || !cfg) return CAI_ERR_INVALID;
  auto fail = [&](const std::string& msg) { g->err = msg + " in " + g->path; return CAI_ERR_INVALID; };
  char arch_buf[64] = {0};
  int found = 0;
  if (cai_gguf_meta_string(g, "general.architecture", arch_buf, sizeof(arch_buf), &found) != CAI_OK) return CAI_ERR_INVALID;
  const std::string arch = arch_buf;
  if (arch != "llama" && arch != "qwen2") {
    g->err = "GGUF import: general.architecture \"" + arch + "\" is not supported (supported: llama, qwen2): " + g->path;
    return CAI_ERR_UNSUPPORTED;
  }
  int st = CAI_OK;
  auto req = [&](const char* suffix, int32_t* out) {
    int64_t v = -1; int f = 0;
    const std::string key = arch + "." + suffix;
    if (cai_gguf_meta_int(g, key.c_str(), &v, &f) != CAI_OK) { st = CAI_ERR_INVALID; return; }
    if (!f || v <= 0 || v > 0x7FFFFFFF) { st = fail("GGUF import: metadata key \"" + key + "\" is missing or not a positive integer"); return; }
    *out = (int32_t)v;
  };
  memset(cfg, 0, sizeof(*cfg));
  int32_t ctx_len = 0;
  req("embedding_length", &cfg->hidden); if (st) return st;
  req("feed_forward_length", &cfg->inter); if (st) return st;
  req("block_count", &cfg->layers); if (st) return st;
  req("attention.head_count", &cfg->heads); if (st) return st;
  req("context_length", &ctx_len); if (st) return st;
  if (max_positions) *max_positions = ctx_len;
  int64_t v = cfg->heads;
  if (cai_gguf_meta_int(g, (arch + ".attention.head_count_kv").c_str(), &v, &found) != CAI_OK) return CAI_ERR_INVALID;
  cfg->kv_heads = (int32_t)v;
  double f = arch == "llama" ? 1e-5 : 1e-6;
  if (cai_gguf_meta_float(g, (arch + ".attention.layer_norm_rms_epsilon").c_str(), &f, &found) != CAI_OK) return CAI_ERR_INVALID;
  cfg->rms_eps = (float)f;
  f = 10000.0;
  if (cai_gguf_meta_float(g, (arch + ".rope.freq_base").c_str(), &f, &found) != CAI_OK) return CAI_ERR_INVALID;
  cfg->rope_theta = (float)f;
  v = 0;
  if (cai_gguf_meta_int(g, (arch + ".attention.key_length").c_str(), &v, &found) != CAI_OK) return CAI_ERR_INVALID;
  cfg->head_dim = (int32_t)v;
  if (arch == "llama") {
    // linear position interpolation is the one scaling mode the reference's llama arm accepts; the decode kernels
    // here rotate by the plain position, so any factor other than 1 is refused rather than silently ignored
    char scaling[32] = "none";
    if (cai_gguf_meta_string(g, "llama.rope.scaling.type", scaling, sizeof(scaling), &found) != CAI_OK) return CAI_ERR_INVALID;
    double factor = 1.0;
    if (std::string(scaling) == "linear") {
      if (cai_gguf_meta_float(g, "llama.rope.scaling.factor", &factor, &found) != CAI_OK) return CAI_ERR_INVALID;
      if (factor < 1) return fail("GGUF import: llama.rope.scaling.factor must be >= 1");
      if (factor != 1.0) { g->err = "GGUF import: RoPE position interpolation (llama.rope.scaling.factor != 1) is not covered by the decode kernels: " + g->path; return CAI_ERR_UNSUPPORTED; }
    } else if (std::string(scaling) != "none") {
      return fail(std::string("GGUF import: llama.rope.scaling.type \"") + scaling + "\" is not supported (supported: none, linear)");
    }
  } else {
    const GGUFMeta* sw = find_meta(g, "qwen2.attention.sliding_window");
    if (sw && sw->i > 0 && (meta_is_int(sw->type)))
      return fail("GGUF import: Qwen2 sliding-window attention is not wired into this importer");
  }
  // vocab: the explicit key, else the embedding rows, else the token list
  v = 0;
  if (cai_gguf_meta_int(g, (arch + ".vocab_size").c_str(), &v, &found) != CAI_OK) return CAI_ERR_INVALID;
  if (v <= 0) {
    auto it = g->tensor_index.find("token_embd.weight");
    if (it != g->tensor_index.end() && g->tensors[(size_t)it->second].ndims == 2) v = g->tensors[(size_t)it->second].shape[0];
    else if (cai_gguf_meta_array_count(g, "tokenizer.ggml.tokens", &v) != CAI_OK) return CAI_ERR_INVALID;
  }
  if (v <= 0) return fail("GGUF import: cannot determine the vocab size");
  cfg->vocab = (int32_t)v;
  cfg->tie_embeddings = g->tensor_index.count("output.weight") ? 0 : 1;
  if (cfg->head_dim <= 0) {
    if (cfg->hidden % cfg->heads) return fail("GGUF import: embedding_length is not divisible by attention.head_count");
    cfg->head_dim = cfg->hidden / cfg->heads;
  }
  cfg->qkv_bias = arch == "qwen2";
  return CAI_OK;
}

int cai_model_load_gguf(cai_ctx* ctx, const char* path, int tp_rank, int tp_size, int quantize_int8, cai_model** out_model,
                        cai_llama_config* out_cfg, int64_t* out_max_positions) {
  CAI_TRY(cai_bind(ctx));
  if (!path || !out_model) return cai_fail(ctx, CAI_ERR_INVALID, "cai_model_load_gguf: null argument");
  *out_model = nullptr;
  cai_gguf* g = nullptr;
  char err[512];
  int st = cai_gguf_open(path, &g, err, sizeof(err));
  if (st != CAI_OK) return cai_fail(ctx, st, "%s", err);
  cai_llama_config cfg;
  st = cai_gguf_llama_config(g, &cfg, out_max_positions);
  if (st != CAI_OK) { st = cai_fail(ctx, st, "%s", g->err.c_str()); cai_gguf_close(g); return st; }
  if (out_cfg) *out_cfg = cfg;
  cai_model* m = nullptr;
  st = cai_model_create(ctx, &cfg, tp_rank, tp_size, &m);
  if (st == CAI_OK && quantize_int8) st = cai_model_set_int8_weights(m, 1);
  const bool qwen2 = cfg.qkv_bias != 0;
  std::vector<uint8_t> raw;
  std::vector<float> f32;
  for (size_t i = 0; i < g->tensors.size() && st == CAI_OK; ++i) {
    const GGUFTensor& t = g->tensors[i];
    std::string hf;
    if (!map_name(t.name, qwen2, &hf)) continue;           // rope_freqs and other tensors the graph has no use for
    if (t.ndims > 2) { st = cai_fail(ctx, CAI_ERR_INVALID, "gguf: tensor \"%s\" has %d dimensions", t.name.c_str(), t.ndims); break; }
    const int64_t rows = t.ndims == 2 ? t.shape[0] : 1, cols = t.ndims == 2 ? t.shape[1] : t.shape[0];
    int bb, be;
    if (!ggml_block(t.type, &bb, &be)) { st = cai_fail(ctx, CAI_ERR_UNSUPPORTED, "gguf: tensor \"%s\" has unsupported type %s", t.name.c_str(), ggml_type_name(t.type)); break; }
    raw.resize((size_t)(t.end - t.begin));
    if (cai_gguf_read_raw(g, (int64_t)i, raw.data(), (int64_t)raw.size()) != CAI_OK) { st = cai_fail(ctx, CAI_ERR_INVALID, "%s", g->err.c_str()); break; }
    // The stored q/k rows are already in the interleaved rotary order the graph runs in: the reference's reader
    // de-interleaves them and its loader interleaves them again (neural/neuralgguf.pas:428-438,
    // neural/neuralpretrained.pas:14792-14812), so the net effect on the resident rows is none.
    if (t.ndims == 1 && t.type != CAI_TYPE_F32) {
      // norm gains and biases are F32 vectors on the device (matrices keep their format; a [q|k|v] or [up|gate] group
      // whose members differ in format is kept as separate matrices by cai_model_upload_tensor)
      f32.resize((size_t)t.n_elems);
      st = gguf_decode_host(ctx, t.type, raw.data(), t.n_elems, f32.data());
      if (st == CAI_OK) st = cai_model_upload_tensor(m, hf.c_str(), CAI_TYPE_F32, f32.data(), rows, cols, 0);
    } else {
      st = cai_model_upload_tensor(m, hf.c_str(), t.type, raw.data(), rows, cols, 0);
    }
  }
  if (st == CAI_OK) st = cai_model_finalize(m);
  cai_gguf_close(g);
  if (st != CAI_OK) { if (m) cai_model_destroy(m); return st; }
  *out_model = m;
  return CAI_OK;
}

}  // extern "C"

// model.cu: tensors of a type the linear kernels do not read directly arrive here and continue as F32
int gguf_upload_decoded(cai_model* m, cai_ctx* ctx, const char* hf_name, int type, const void* data_host, int64_t rows, int64_t cols,
                        int interleave_head_dim) {
  std::vector<float> f32((size_t)rows * (size_t)cols);
  CAI_TRY(gguf_decode_host(ctx, type, data_host, rows * cols, f32.data()));
  return cai_model_upload_tensor(m, hf_name, CAI_TYPE_F32, f32.data(), rows, cols, interleave_head_dim);
}

bool gguf_type_needs_decode(int type) {
  // Q4_K, Q5_K and Q6_K stay resident as raw super-blocks (the K-quant GEMV reads them); the others become fp32
  return type == 3 || type == 6 || type == 7 || type == 10 || type == 11;
}
