// Weight loading: a safetensors reader (mmap + header index) and the checkpoint loaders of the
// executors. Counterparts in the reference:
//   Reader::open / get / names          crates/loader/src/safetensors.rs:44-197 (mmap, upstream header
//                                       validation, per-tensor byte ranges, archive ordering by offset)
//   check_mmap_not_truncated            crates/loader/src/lib.rs:229-246 (re-stat before every access)
//   StellaWeights::load, load_layer     crates/encoders/src/stella.rs:123-166, :320-400 (exact tensor
//                                       count, per-name F32 + shape checks)
//   StellaModel::load, load_dense_head  crates/embed/src/stella.rs:138-201, :380-443
// The header rules restated here are those of the safetensors format the reference's parser enforces
// (safetensors 0.7 `SafeTensors::read_metadata`): an 8-byte little-endian header length, a JSON object
// of name -> {dtype, shape, data_offsets}, tensors laid out back to back from offset 0 without holes
// or overlaps up to the end of the file, and every byte range equal to the element size times the
// product of the shape.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cuda_runtime.h>

#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "logismos_kernels.h"
#include "logismos_model.h"

namespace lgm { void set_error(const std::string& s); }

namespace {

using lgm::set_error;

struct Entry {
  int dtype = 0;
  std::vector<int64_t> shape;
  size_t start = 0, end = 0;  // absolute byte range in the mapping
};

struct Reader {
  std::string path;
  const uint8_t* map = nullptr;
  size_t len = 0;
  size_t data_start = 0;
  std::vector<std::string> ordering;  // by on-disk offset
  std::map<std::string, Entry> index;
  ~Reader() {
    if (map) munmap(const_cast<uint8_t*>(map), len);
  }
};

// ---- a JSON reader sufficient for the safetensors header ------------------------------------
struct Json {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  bool string(std::string& out) {
    ws();
    if (p >= e || *p != '"') return ok = false;
    ++p;
    out.clear();
    while (p < e && *p != '"') {
      if (*p == '\\') {
        if (++p >= e) return ok = false;
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {  // \uXXXX -> UTF-8 (basic plane; surrogate pairs kept as two code units)
            if (e - p < 5) return ok = false;
            unsigned v = 0;
            for (int i = 1; i <= 4; ++i) {
              const char c = p[i];
              v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 32) >= 'a' && (c | 32) <= 'f' ? (c | 32) - 'a' + 10 : 0);
            }
            p += 4;
            if (v < 0x80) out += (char)v;
            else if (v < 0x800) { out += (char)(0xc0 | (v >> 6)); out += (char)(0x80 | (v & 63)); }
            else { out += (char)(0xe0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 63)); out += (char)(0x80 | (v & 63)); }
            break;
          }
          default: out += *p;  // \" \\ \/
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= e) return ok = false;
    ++p;
    return true;
  }
  bool uint(uint64_t& v) {
    ws();
    if (p >= e || *p < '0' || *p > '9') return ok = false;
    v = 0;
    while (p < e && *p >= '0' && *p <= '9') {
      if (v > (UINT64_MAX - 9) / 10) return ok = false;
      v = v * 10 + (uint64_t)(*p++ - '0');
    }
    return true;
  }
  // skips any value (used for __metadata__)
  bool skip() {
    ws();
    if (p >= e) return ok = false;
    if (*p == '"') { std::string s; return string(s); }
    if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      const bool obj = *p == '{';
      ++p;
      if (eat(close)) return true;
      for (;;) {
        if (obj) { std::string k; if (!string(k) || !eat(':')) return ok = false; }
        if (!skip()) return false;
        if (eat(',')) continue;
        return eat(close) ? true : (ok = false);
      }
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;  // number, true, false, null
    return true;
  }
};

struct DtypeInfo { const char* name; int code; size_t size; };
// the dtypes the reference maps (crates/loader/src/safetensors.rs:199-217); codes follow logismos_model.h
const DtypeInfo kDtypes[] = {{"F32", LG_DT_F32, 4},       {"F16", LG_DT_F16, 2},         {"BF16", LG_DT_BF16, 2}, {"I32", LG_DT_I32, 4},
                             {"I8", LG_DT_I8, 1},         {"U8", LG_DT_U8, 1},           {"F8_E4M3", LG_DT_F8E4M3, 1},
                             {"F8_E5M2", LG_DT_F8E5M2, 1}};
// valid in the format but not mapped by the reference: rejected per tensor with a message
const DtypeInfo kUnmapped[] = {{"BOOL", -1, 1}, {"U16", -1, 2}, {"I16", -1, 2}, {"U32", -1, 4}, {"I64", -1, 8}, {"U64", -1, 8}, {"F64", -1, 8}};

uint32_t fail(uint32_t code, const std::string& msg) {
  set_error(msg);
  return code;
}

uint32_t open_reader(const char* path, Reader** out) {
  *out = nullptr;
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) return fail(LG_EMB_IO, std::string("open ") + path + ": " + std::strerror(errno));
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) {
    ::close(fd);
    return fail(LG_EMB_IO, std::string(path) + ": not a safetensors file (shorter than its 8-byte header length)");
  }
  Reader* r = new Reader();
  r->path = path;
  r->len = (size_t)st.st_size;
  void* m = mmap(nullptr, r->len, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) { delete r; return fail(LG_EMB_IO, std::string("mmap ") + path + ": " + std::strerror(errno)); }
  r->map = (const uint8_t*)m;
  uint64_t hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | r->map[i];
  if (hlen > 100000000ull || hlen > r->len - 8) { delete r; return fail(LG_EMB_IO, std::string(path) + ": safetensors header length is invalid"); }
  r->data_start = 8 + (size_t)hlen;
  Json j{(const char*)r->map + 8, (const char*)r->map + 8 + hlen};
  if (!j.eat('{')) { delete r; return fail(LG_EMB_IO, std::string(path) + ": safetensors header is not a JSON object"); }
  bool first = true;
  while (!j.eat('}')) {
    if (!first && !j.eat(',')) { j.ok = false; break; }
    first = false;
    std::string name;
    if (!j.string(name) || !j.eat(':')) { j.ok = false; break; }
    if (name == "__metadata__") { if (!j.skip()) break; continue; }
    Entry en;
    std::string dt;
    uint64_t o0 = 0, o1 = 0;
    bool have_dt = false, have_shape = false, have_off = false;
    if (!j.eat('{')) { j.ok = false; break; }
    bool f2 = true;
    while (!j.eat('}')) {
      if (!f2 && !j.eat(',')) { j.ok = false; break; }
      f2 = false;
      std::string k;
      if (!j.string(k) || !j.eat(':')) { j.ok = false; break; }
      if (k == "dtype") { have_dt = j.string(dt); }
      else if (k == "shape") {
        if (!j.eat('[')) { j.ok = false; break; }
        if (!j.eat(']')) {
          for (;;) {
            uint64_t v;
            if (!j.uint(v)) break;
            en.shape.push_back((int64_t)v);
            if (j.eat(',')) continue;
            if (!j.eat(']')) j.ok = false;
            break;
          }
        }
        have_shape = j.ok;
      } else if (k == "data_offsets") {
        have_off = j.eat('[') && j.uint(o0) && j.eat(',') && j.uint(o1) && j.eat(']');
        if (!have_off) j.ok = false;
      } else if (!j.skip()) break;
      if (!j.ok) break;
    }
    if (!j.ok) break;
    if (!have_dt || !have_shape || !have_off) { delete r; return fail(LG_EMB_IO, std::string(path) + ": tensor `" + name + "` lacks dtype, shape or data_offsets"); }
    size_t esz = 0;
    en.dtype = -2;
    for (const DtypeInfo& d : kDtypes) if (dt == d.name) { en.dtype = d.code; esz = d.size; }
    for (const DtypeInfo& d : kUnmapped) if (dt == d.name) { en.dtype = -1; esz = d.size; }
    if (en.dtype == -2) { delete r; return fail(LG_EMB_IO, std::string(path) + ": tensor `" + name + "` has unknown dtype " + dt); }
    if (en.dtype == -1) { delete r; return fail(LG_EMB_IO, "tensor `" + name + "` uses unmapped safetensors dtype " + dt); }
    unsigned __int128 n = 1;
    for (int64_t s : en.shape) { n *= (unsigned __int128)s; if (n > (unsigned __int128)1 << 62) break; }
    if (o1 < o0 || (unsigned __int128)(o1 - o0) != n * esz) {
      delete r;
      return fail(LG_EMB_IO, std::string(path) + ": tensor `" + name + "`: byte range does not match dtype x shape");
    }
    en.start = r->data_start + (size_t)o0;
    en.end = r->data_start + (size_t)o1;
    if (en.end > r->len || en.start > en.end) { delete r; return fail(LG_EMB_IO, std::string(path) + ": tensor `" + name + "` lies outside the file"); }
    if (r->index.count(name)) { delete r; return fail(LG_EMB_IO, std::string(path) + ": tensor `" + name + "` appears twice"); }
    r->index[name] = en;
    r->ordering.push_back(name);
  }
  if (!j.ok) { delete r; return fail(LG_EMB_IO, std::string(path) + ": malformed safetensors header"); }
  // archive ordering = by offset; the data region must be covered exactly, back to back
  std::stable_sort(r->ordering.begin(), r->ordering.end(), [&](const std::string& a, const std::string& b) {
    const Entry &x = r->index[a], &y = r->index[b];
    return x.start != y.start ? x.start < y.start : a < b;
  });
  size_t at = r->data_start;
  for (const std::string& n : r->ordering) {
    const Entry& en = r->index[n];
    if (en.start != at) {
      const std::string msg = std::string(path) + ": tensor `" + n + "` leaves a hole or overlaps its neighbour";  // n dies with r
      delete r;
      return fail(LG_EMB_IO, msg);
    }
    at = en.end;
  }
  if (at != r->len) { delete r; return fail(LG_EMB_IO, std::string(path) + ": tensor data does not end at the end of the file"); }
  *out = r;
  return LG_EMB_OK;
}

// crates/loader/src/lib.rs:229-246
uint32_t check_not_truncated(const Reader* r) {
  struct stat st;
  if (stat(r->path.c_str(), &st) != 0) return fail(LG_EMB_IO, "stat " + r->path + ": " + std::strerror(errno));
  if ((size_t)st.st_size != r->len) {
    char b[160];
    std::snprintf(b, sizeof(b), ": mapped %zu bytes, the file now has %lld (changed after it was opened)", r->len, (long long)st.st_size);
    return fail(LG_EMB_IO, r->path + b);
  }
  return LG_EMB_OK;
}

uint32_t get_view(const Reader* r, const char* name, lg_tensor_view_t* out) {
  if (uint32_t rc = check_not_truncated(r)) return rc;
  auto it = r->index.find(name);
  if (it == r->index.end()) return fail(LG_EMB_IO, std::string("tensor not found: ") + name);
  const Entry& en = it->second;
  if (en.shape.size() > 8) return fail(LG_EMB_IO, std::string(name) + ": rank above 8");
  out->dtype = en.dtype;
  out->rank = (int32_t)en.shape.size();
  for (int i = 0; i < 8; ++i) out->shape[i] = i < out->rank ? en.shape[i] : 0;
  out->data = r->map + en.start;
  out->nbytes = en.end - en.start;
  return LG_EMB_OK;
}

// read_f32 of crates/encoders/src/stella.rs:376-400: F32 and the exact shape, else a layout error
uint32_t want_f32(const Reader* r, const std::string& name, std::initializer_list<int64_t> shape, const float** out) {
  lg_tensor_view_t v;
  if (uint32_t rc = get_view(r, name.c_str(), &v)) return rc;
  if (v.dtype != LG_DT_F32) return fail(LG_EMB_COMPUTE, name + ": expected F32");
  bool same = v.rank == (int32_t)shape.size();
  int i = 0;
  for (int64_t s : shape) { if (same && v.shape[i] != s) same = false; ++i; }
  if (!same) {
    std::string got = "[", exp = "[";
    for (int k = 0; k < v.rank; ++k) got += (k ? ", " : "") + std::to_string(v.shape[k]);
    int k = 0;
    for (int64_t s : shape) exp += (k++ ? ", " : "") + std::to_string(s);
    return fail(LG_EMB_COMPUTE, name + ": expected shape " + exp + "], got " + got + "]");
  }
  if (((uintptr_t)v.data & 3) != 0) return fail(LG_EMB_COMPUTE, name + ": data is not 4-byte aligned in the file");
  *out = (const float*)v.data;
  return LG_EMB_OK;
}

}  // namespace

extern "C" {

uint32_t lg_safetensors_open(const char* path, void** reader) {
  if (!path || !reader) return fail(LG_EMB_COMPUTE, "null argument");
  Reader* r = nullptr;
  const uint32_t rc = open_reader(path, &r);
  *reader = r;
  return rc;
}

void lg_safetensors_close(void* reader) { delete static_cast<Reader*>(reader); }

int32_t lg_safetensors_len(const void* reader) { return (int32_t)static_cast<const Reader*>(reader)->ordering.size(); }

const char* lg_safetensors_name(const void* reader, int32_t i) {
  const Reader* r = static_cast<const Reader*>(reader);
  return (i >= 0 && (size_t)i < r->ordering.size()) ? r->ordering[(size_t)i].c_str() : nullptr;
}

uint64_t lg_safetensors_data_region_start(const void* reader) { return static_cast<const Reader*>(reader)->data_start; }

uint32_t lg_safetensors_get(const void* reader, const char* name, lg_tensor_view_t* out) {
  if (!reader || !name || !out) return fail(LG_EMB_COMPUTE, "null argument");
  return get_view(static_cast<const Reader*>(reader), name, out);
}

uint32_t lg_stella_load(int32_t device, const char* root, const lg_stella_config_t* cfg, void** model) {
  if (!root || !cfg || !model) return fail(LG_EMB_COMPUTE, "null argument");
  *model = nullptr;
  const lg_stella_config_t& c = *cfg;
  if (c.n_heads <= 0 || c.n_layers < 0 || c.n_dims <= 0 || c.n_dims > 8) return fail(LG_EMB_COMPUTE, "lg_stella_load: bad config");
  const std::string dir(root);
  Reader* r = nullptr;
  if (uint32_t rc = open_reader((dir + "/model.safetensors").c_str(), &r)) return rc;
  struct Guard { std::vector<Reader*> rs; ~Guard() { for (Reader* x : rs) delete x; } } guard;
  guard.rs.push_back(r);
  // the archive must hold exactly the tensors this model reads (crates/encoders/src/stella.rs:126-145)
  const size_t expected = 2 + (size_t)c.n_layers * 12;
  if (r->ordering.size() != expected)
    return fail(LG_EMB_COMPUTE, "expected " + std::to_string(expected) + " tensors in stella archive, got " + std::to_string(r->ordering.size()));
  const int64_t H = c.hidden, I = c.intermediate, KV = (int64_t)c.n_kv_heads * (c.hidden / c.n_heads);
  lg_stella_weights_t w{};
  std::vector<lg_stella_layer_weights_t> layers((size_t)c.n_layers);
  if (uint32_t rc = want_f32(r, "model.embed_tokens.weight", {c.vocab, H}, &w.tok_embed)) return rc;
  if (uint32_t rc = want_f32(r, "model.norm.weight", {H}, &w.final_norm)) return rc;
  for (int i = 0; i < c.n_layers; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    lg_stella_layer_weights_t& L = layers[(size_t)i];
    uint32_t rc = 0;
    (rc = want_f32(r, p + "input_layernorm.weight", {H}, &L.norm1)) || (rc = want_f32(r, p + "post_attention_layernorm.weight", {H}, &L.norm2)) ||
        (rc = want_f32(r, p + "self_attn.q_proj.weight", {H, H}, &L.wq)) || (rc = want_f32(r, p + "self_attn.q_proj.bias", {H}, &L.bq)) ||
        (rc = want_f32(r, p + "self_attn.k_proj.weight", {KV, H}, &L.wk)) || (rc = want_f32(r, p + "self_attn.k_proj.bias", {KV}, &L.bk)) ||
        (rc = want_f32(r, p + "self_attn.v_proj.weight", {KV, H}, &L.wv)) || (rc = want_f32(r, p + "self_attn.v_proj.bias", {KV}, &L.bv)) ||
        (rc = want_f32(r, p + "self_attn.o_proj.weight", {H, H}, &L.wo)) || (rc = want_f32(r, p + "mlp.gate_proj.weight", {I, H}, &L.w_gate)) ||
        (rc = want_f32(r, p + "mlp.up_proj.weight", {I, H}, &L.w_up)) || (rc = want_f32(r, p + "mlp.down_proj.weight", {H, I}, &L.w_down));
    if (rc) return rc;
  }
  w.layers = layers.data();
  // supported dims sorted, the default is 1024 when that head is loaded, else the smallest
  // (crates/embed/src/stella.rs:143-163); the model takes its default from dims[0]
  lg_stella_config_t cc = c;
  std::sort(cc.dims, cc.dims + cc.n_dims);
  for (int d = 0; d < cc.n_dims; ++d)
    if (cc.dims[d] == 1024) std::rotate(cc.dims, cc.dims + d, cc.dims + d + 1);
  // dense heads: <root>/2_Dense_<dim>/model.safetensors with linear.weight [dim, hidden], linear.bias [dim]
  // (crates/embed/src/stella.rs:380-443)
  for (int d = 0; d < cc.n_dims; ++d) {
    Reader* hr = nullptr;
    const std::string folder = "2_Dense_" + std::to_string(cc.dims[d]);
    if (uint32_t rc = open_reader((dir + "/" + folder + "/model.safetensors").c_str(), &hr)) return rc;
    guard.rs.push_back(hr);
    lg_tensor_view_t wv, bv;
    if (uint32_t rc = get_view(hr, "linear.weight", &wv)) return rc;
    if (uint32_t rc = get_view(hr, "linear.bias", &bv)) return rc;
    if (wv.dtype != LG_DT_F32 || bv.dtype != LG_DT_F32) return fail(LG_EMB_IO, "dense head " + folder + ": expected F32");
    if (wv.rank != 2 || wv.shape[0] != cc.dims[d] || wv.shape[1] != H)
      return fail(LG_EMB_IO, "dense head " + folder + ": expected weight shape [" + std::to_string(cc.dims[d]) + ", " + std::to_string(H) + "]");
    if (bv.rank != 1 || bv.shape[0] != cc.dims[d]) return fail(LG_EMB_IO, "dense head " + folder + ": expected bias shape [" + std::to_string(cc.dims[d]) + "]");
    w.head_w[d] = (const float*)wv.data;
    w.head_b[d] = (const float*)bv.data;
  }
  return lg_stella_create(device, &cc, &w, model);
}

// The int4 decoder from a Qwen2-style checkpoint (fp32 tensors under the names of
// crates/encoders/src/stella.rs:326-349 plus lm_head.weight [vocab, hidden]; when that tensor is absent
// the head is tied to the embedding): every matrix is quantised to int4 group-32 ON THE DEVICE
// (logismos_launch_quantize_int4_g32) and handed to lg_decoder_create. No reference counterpart beyond
// the tensor accounting: the reference has no quantiser and no decoder.
uint32_t lg_decoder_load(int32_t device, const char* path, const lg_decoder_config_t* cfg, void** model) {
  if (!path || !cfg || !model) return fail(LG_EMB_COMPUTE, "null argument");
  *model = nullptr;
  const lg_decoder_config_t& c = *cfg;
  if (c.n_heads <= 0 || c.n_layers < 0 || c.hidden % 32 || c.intermediate % 32) return fail(LG_EMB_COMPUTE, "lg_decoder_load: bad config");
  Reader* r = nullptr;
  if (uint32_t rc = open_reader(path, &r)) return rc;
  struct Guard { Reader* r; ~Guard() { delete r; } } guard{r};
  const bool tied = r->index.find("lm_head.weight") == r->index.end();
  const size_t expected = 2 + (tied ? 0 : 1) + (size_t)c.n_layers * 12;
  if (r->ordering.size() != expected)
    return fail(LG_EMB_COMPUTE, "expected " + std::to_string(expected) + " tensors in decoder archive, got " + std::to_string(r->ordering.size()));
  if (cudaSetDevice(device) != cudaSuccess) return fail(LG_EMB_COMPUTE, "cudaSetDevice failed");
  const int64_t H = c.hidden, I = c.intermediate, KV = (int64_t)c.n_kv_heads * (c.hidden / c.n_heads);
  struct QHost { std::vector<uint8_t> codes; std::vector<uint16_t> scales; };
  std::vector<QHost> store;
  store.reserve((size_t)c.n_layers * 7 + 1);
  size_t scratch_elems = (size_t)c.vocab * H;
  if ((size_t)I * H > scratch_elems) scratch_elems = (size_t)I * H;
  float* d_w = nullptr;
  uint8_t* d_codes = nullptr;
  uint16_t* d_scales = nullptr;
  struct DevGuard { float** a; uint8_t** b; uint16_t** c; ~DevGuard() { if (*a) cudaFree(*a); if (*b) cudaFree(*b); if (*c) cudaFree(*c); } } dg{&d_w, &d_codes, &d_scales};
  if (cudaMalloc(&d_w, scratch_elems * 4) != cudaSuccess || cudaMalloc(&d_codes, scratch_elems / 2) != cudaSuccess ||
      cudaMalloc(&d_scales, scratch_elems / 32 * 2) != cudaSuccess)
    return fail(LG_EMB_COMPUTE, "lg_decoder_load: device scratch allocation failed");
  auto quant = [&](const std::string& name, int64_t n, int64_t k, lg_int4_matrix_t* out) -> uint32_t {
    const float* src = nullptr;
    if (uint32_t rc = want_f32(r, name, {n, k}, &src)) return rc;
    store.emplace_back();
    QHost& q = store.back();
    q.codes.resize((size_t)n * k / 2);
    q.scales.resize((size_t)n * k / 32);
    if (cudaMemcpy(d_w, src, (size_t)n * k * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
        logismos_launch_quantize_int4_g32(d_w, d_codes, d_scales, (int32_t)n, (int32_t)k, nullptr) != 0 ||
        cudaMemcpy(q.codes.data(), d_codes, q.codes.size(), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(q.scales.data(), d_scales, q.scales.size() * 2, cudaMemcpyDeviceToHost) != cudaSuccess)
      return fail(LG_EMB_COMPUTE, name + ": quantisation on the device failed");
    out->codes = q.codes.data();
    out->scales = q.scales.data();
    return LG_EMB_OK;
  };
  lg_decoder_weights_t w{};
  std::vector<lg_decoder_layer_weights_t> layers((size_t)c.n_layers);
  if (uint32_t rc = want_f32(r, "model.embed_tokens.weight", {c.vocab, H}, &w.tok_embed)) return rc;
  if (uint32_t rc = want_f32(r, "model.norm.weight", {H}, &w.final_norm)) return rc;
  if (uint32_t rc = quant(tied ? "model.embed_tokens.weight" : "lm_head.weight", c.vocab, H, &w.lm_head)) return rc;
  for (int i = 0; i < c.n_layers; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    lg_decoder_layer_weights_t& L = layers[(size_t)i];
    uint32_t rc = 0;
    (rc = want_f32(r, p + "input_layernorm.weight", {H}, &L.norm1)) || (rc = want_f32(r, p + "post_attention_layernorm.weight", {H}, &L.norm2)) ||
        (rc = want_f32(r, p + "self_attn.q_proj.bias", {H}, &L.bq)) || (rc = want_f32(r, p + "self_attn.k_proj.bias", {KV}, &L.bk)) ||
        (rc = want_f32(r, p + "self_attn.v_proj.bias", {KV}, &L.bv)) || (rc = quant(p + "self_attn.q_proj.weight", H, H, &L.wq)) ||
        (rc = quant(p + "self_attn.k_proj.weight", KV, H, &L.wk)) || (rc = quant(p + "self_attn.v_proj.weight", KV, H, &L.wv)) ||
        (rc = quant(p + "self_attn.o_proj.weight", H, H, &L.wo)) || (rc = quant(p + "mlp.gate_proj.weight", I, H, &L.w_gate)) ||
        (rc = quant(p + "mlp.up_proj.weight", I, H, &L.w_up)) || (rc = quant(p + "mlp.down_proj.weight", H, I, &L.w_down));
    if (rc) return rc;
  }
  w.layers = layers.data();
  return lg_decoder_create(device, cfg, &w, model);
}

}  // extern "C"
