// Weight ingestion for the quantized MOSS-Image DiT: one ComfyUI-layout safetensors file -> device tensors in the form
// the block kernels consume, validated as untrusted input before any byte of a tensor is read.
//
// What the reference's reader accepts for this path (src/weights/quant/quant_model.h:1-45, quant_model.cpp:205-285,
// 354-380) and this one reads:
//   names       official DiT names, bare or under "diffusion_model." / "model.diffusion_model."
//   configs     per module, the `<module>.comfy_quant` U8 tensor (JSON, fields also under "params") or the legacy
//               `_quantization_metadata` header key ({"layers": {module: config}})
//   int8_tensorwise + convrot (group 256)   <m>.weight I8 [N, K], <m>.weight_scale F32 [N] | [N, 1] | scalar
//   convrot_w4a4                            <m>.weight I8 [N, K/2] (signed nibbles, even column low), <m>.weight_scale F32 [N]
//   asym_w4a8_int8                          <m>.weight I8 [N, K/2], <m>.weight_s_rel F8_E4M3 | U8 [N, K/group],
//                                           <m>.weight_s_channel F32 [N], optional <m>.weight_codebook F32 [16]
//   layers.N.proj.qkv ([3 D, D]) or proj.q / proj.k / proj.v (stacked here in that order), proj.o, proj.ffn_up_gate
//   ([2 F, D], stored [hidden | gate]), proj.ffn_down ([D, F]); norm1, norm2 (BF16 [D]), q_norm, k_norm (BF16 [128]).
//   Outside the blocks (moss_dit.cpp:753-761), when present: video_embedder, time_embedding.0 / .2,
//   shared_block_modulation, video_head_modulation, final_norm_video, final_linear_video.
// Refused, each with a message that names the module: plain INT8 without rotation, a rotation group other than 256,
// w6a8_int8 and nvfp4, q / k / v in different formats, a model that mixes tiers, scales that are not finite and > 0,
// shapes that are not the DiT's. Where the reference decodes the 4-bit formats to INT8 on the CPU at load, the packed
// bytes go to the device as stored and the block's tier decodes them (B2_TIER_W4A4_VIA_INT8, B2_TIER_W4A8).
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <system_error>
#include <thread>
#include <vector>

#include "common.cuh"

namespace b2 {
namespace {

constexpr std::uint64_t kMaxHeaderBytes = std::uint64_t{16} << 20;  // as the reference's reader (safetensors.h)
constexpr std::size_t kMaxTensors = 65536, kMaxConfigBytes = 4096;
constexpr std::int64_t kDim = 3072, kHeadDim = 128, kLatent = 128, kFreq = 256;

struct LoadError {
  std::string what;
};
[[noreturn]] void fail(const std::string& msg) { throw LoadError{msg}; }

// ------------------------------------------------------------------------------------------------ a small JSON reader

struct Json {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool b = false;
  double num = 0;
  bool integral = false;
  std::int64_t inum = 0;
  std::string str;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> fields;
  const Json* find(const std::string& key) const {
    for (const auto& f : fields) {
      if (f.first == key) return &f.second;
    }
    return nullptr;
  }
};

class JsonParser {
 public:
  JsonParser(const char* p, std::size_t n) : p_(p), end_(p + n) {}
  Json parse() {
    Json v = value(0);
    skip();
    if (p_ != end_) fail("JSON: trailing bytes");
    return v;
  }

 private:
  const char* p_;
  const char* end_;
  void skip() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  char peek() {
    skip();
    if (p_ >= end_) fail("JSON: unexpected end");
    return *p_;
  }
  void expect(char c) {
    if (peek() != c) fail(std::string("JSON: expected '") + c + "'");
    ++p_;
  }
  std::string string() {
    expect('"');
    std::string s;
    while (true) {
      if (p_ >= end_) fail("JSON: unterminated string");
      const char c = *p_++;
      if (c == '"') return s;
      if (static_cast<unsigned char>(c) < 0x20) fail("JSON: control character in a string");
      if (c != '\\') {
        s.push_back(c);
        continue;
      }
      if (p_ >= end_) fail("JSON: unterminated escape");
      const char e = *p_++;
      switch (e) {
        case '"': case '\\': case '/': s.push_back(e); break;
        case 'b': s.push_back('\b'); break;
        case 'f': s.push_back('\f'); break;
        case 'n': s.push_back('\n'); break;
        case 'r': s.push_back('\r'); break;
        case 't': s.push_back('\t'); break;
        case 'u': {
          if (end_ - p_ < 4) fail("JSON: short \\u escape");
          unsigned cp = 0;
          for (int i = 0; i < 4; ++i) {
            const char h = *p_++;
            cp = cp * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 1000);
          }
          if (cp > 0xFFFF) fail("JSON: bad \\u escape");
          // Names and configs are ASCII; anything else is kept as UTF-8 of the code unit.
          if (cp < 0x80) s.push_back(static_cast<char>(cp));
          else if (cp < 0x800) s.push_back(static_cast<char>(0xC0 | (cp >> 6))), s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          else s.push_back(static_cast<char>(0xE0 | (cp >> 12))), s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))), s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          break;
        }
        default: fail("JSON: unknown escape");
      }
    }
  }
  Json value(int depth) {
    if (depth > 16) fail("JSON: nested too deeply");
    Json v;
    const char c = peek();
    if (c == '{') {
      ++p_;
      v.kind = Json::kObject;
      if (peek() == '}') {
        ++p_;
        return v;
      }
      while (true) {
        std::string key = (skip(), string());
        expect(':');
        v.fields.emplace_back(std::move(key), value(depth + 1));
        if (v.fields.size() > 4 * kMaxTensors) fail("JSON: too many fields");
        if (peek() == ',') {
          ++p_;
          continue;
        }
        expect('}');
        return v;
      }
    }
    if (c == '[') {
      ++p_;
      v.kind = Json::kArray;
      if (peek() == ']') {
        ++p_;
        return v;
      }
      while (true) {
        v.items.push_back(value(depth + 1));
        if (peek() == ',') {
          ++p_;
          continue;
        }
        expect(']');
        return v;
      }
    }
    if (c == '"') {
      v.kind = Json::kString;
      v.str = string();
      return v;
    }
    const auto word = [&](const char* w) {
      const std::size_t n = std::strlen(w);
      if (static_cast<std::size_t>(end_ - p_) < n || std::memcmp(p_, w, n) != 0) return false;
      p_ += n;
      return true;
    };
    if (word("true")) return v.kind = Json::kBool, v.b = true, v;
    if (word("false")) return v.kind = Json::kBool, v;
    if (word("null")) return v;
    const char* start = p_;
    if (p_ < end_ && *p_ == '-') ++p_;
    bool digits = false, frac = false;
    while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '+' || *p_ == '-')) {
      digits = digits || (*p_ >= '0' && *p_ <= '9');
      frac = frac || *p_ == '.' || *p_ == 'e' || *p_ == 'E';
      ++p_;
    }
    if (!digits) fail("JSON: unexpected character");
    const std::string text(start, p_);
    v.kind = Json::kNumber;
    try {
      v.num = std::stod(text);
      if (!frac && text.size() <= 18) v.integral = true, v.inum = std::stoll(text);
    } catch (...) {
      fail("JSON: bad number '" + text + "'");
    }
    return v;
  }
};

// ------------------------------------------------------------------------------------------------ the container

enum class DT { kU8, kI8, kF8E4M3, kF16, kBF16, kF32, kOther };
std::size_t dt_size(DT t, const std::string& name) {
  switch (t) {
    case DT::kU8: case DT::kI8: case DT::kF8E4M3: return 1;
    case DT::kF16: case DT::kBF16: return 2;
    case DT::kF32: return 4;
    default: break;
  }
  if (name == "BOOL" || name == "F8_E5M2" || name == "F8_E8M0") return 1;
  if (name == "I16" || name == "U16") return 2;
  if (name == "I32" || name == "U32") return 4;
  if (name == "I64" || name == "U64" || name == "F64") return 8;
  return 0;
}
DT parse_dt(const std::string& s) {
  if (s == "U8") return DT::kU8;
  if (s == "I8") return DT::kI8;
  if (s == "F8_E4M3") return DT::kF8E4M3;
  if (s == "F16") return DT::kF16;
  if (s == "BF16") return DT::kBF16;
  if (s == "F32") return DT::kF32;
  return DT::kOther;
}

struct Entry {
  DT dtype = DT::kOther;
  std::string dtype_name;
  std::vector<std::int64_t> shape;
  std::uint64_t offset = 0, nbytes = 0;  // absolute file offset
  std::int64_t numel() const {
    std::int64_t n = 1;
    for (std::int64_t d : shape) n *= d;
    return n;
  }
  std::string describe() const {
    std::string s = dtype_name + " [";
    for (std::size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
  }
};

struct File {
  int fd = -1;
  std::uint64_t size = 0;
  std::map<std::string, Entry> tensors;  // canonical names (prefix stripped)
  std::map<std::string, std::string> metadata;
  ~File() {
    if (fd >= 0) ::close(fd);
  }
  // false (and *bad = the offset) on a short read.
  bool read_piece(std::uint64_t offset, char* out, std::size_t n, std::uint64_t* bad) const {
    while (n > 0) {
      const ssize_t got = ::pread(fd, out, n, static_cast<off_t>(offset));
      if (got <= 0) {
        *bad = offset;
        return false;
      }
      out += got, offset += static_cast<std::uint64_t>(got), n -= static_cast<std::size_t>(got);
    }
    return true;
  }
  // A large read is split over four threads: one thread copying out of the page cache moves 4-5 GB/s, far below what the
  // copy to the device behind it takes.
  void read(std::uint64_t offset, void* dst, std::size_t n) const {
    char* out = static_cast<char*>(dst);
    constexpr int kPieces = 4;
    bool ok[kPieces] = {true, true, true, true};
    std::uint64_t bad[kPieces] = {0, 0, 0, 0};
    if (n < (std::size_t{8} << 20)) {
      ok[0] = read_piece(offset, out, n, &bad[0]);
    } else {
      const std::size_t per = (n / kPieces + 4095) & ~std::size_t{4095};
      std::vector<std::thread> workers;
      for (int i = 1; i < kPieces; ++i) {
        const std::size_t at = std::min(n, per * static_cast<std::size_t>(i)), len = std::min(n, per * static_cast<std::size_t>(i + 1)) - at;
        if (len == 0) continue;
        try {
          workers.emplace_back([=, &ok, &bad] { ok[i] = read_piece(offset + at, out + at, len, &bad[i]); });
        } catch (const std::system_error&) {
          ok[i] = read_piece(offset + at, out + at, len, &bad[i]);
        }
      }
      ok[0] = read_piece(offset, out, std::min(n, per), &bad[0]);
      for (std::thread& w : workers) w.join();
    }
    for (int i = 0; i < kPieces; ++i) {
      if (!ok[i]) fail("short read at byte " + std::to_string(bad[i]));
    }
  }
  const Entry* find(const std::string& name) const {
    const auto it = tensors.find(name);
    return it == tensors.end() ? nullptr : &it->second;
  }
};

std::string canonical(std::string name) {
  for (const char* p : {"model.diffusion_model.", "diffusion_model."}) {
    const std::size_t n = std::strlen(p);
    if (name.compare(0, n, p) == 0) return name.substr(n);
  }
  return name;
}

void open_file(const char* path, File* f) {
  f->fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (f->fd < 0) fail("cannot open the file");
  struct stat st {};
  if (::fstat(f->fd, &st) != 0 || !S_ISREG(st.st_mode)) fail("not a regular file");
  f->size = static_cast<std::uint64_t>(st.st_size);
  if (f->size < 8) fail("shorter than a safetensors header");
  unsigned char len8[8];
  f->read(0, len8, 8);
  std::uint64_t hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | len8[i];
  if (hlen < 2 || hlen > kMaxHeaderBytes || hlen > f->size - 8) fail("header length " + std::to_string(hlen) + " is out of range");
  std::string text(static_cast<std::size_t>(hlen), '\0');
  f->read(8, text.data(), text.size());
  const Json root = JsonParser(text.data(), text.size()).parse();
  if (root.kind != Json::kObject) fail("the header is not a JSON object");
  const std::uint64_t data_start = 8 + hlen, data_bytes = f->size - data_start;
  for (const auto& [raw_name, v] : root.fields) {
    if (raw_name == "__metadata__") {
      if (v.kind != Json::kObject) fail("__metadata__ is not an object");
      for (const auto& [k, mv] : v.fields) {
        if (mv.kind == Json::kString) f->metadata[k] = mv.str;
      }
      continue;
    }
    if (f->tensors.size() >= kMaxTensors) fail("more than " + std::to_string(kMaxTensors) + " tensors");
    const Json *dt = v.find("dtype"), *sh = v.find("shape"), *off = v.find("data_offsets");
    if (v.kind != Json::kObject || dt == nullptr || dt->kind != Json::kString || sh == nullptr || sh->kind != Json::kArray ||
        off == nullptr || off->kind != Json::kArray || off->items.size() != 2) {
      fail("tensor '" + raw_name + "': needs dtype, shape and data_offsets");
    }
    Entry e;
    e.dtype_name = dt->str;
    e.dtype = parse_dt(dt->str);
    const std::size_t esize = dt_size(e.dtype, dt->str);
    if (esize == 0) fail("tensor '" + raw_name + "': unknown dtype '" + dt->str + "'");
    if (sh->items.size() > 8) fail("tensor '" + raw_name + "': rank above 8");
    std::uint64_t count = 1;
    for (const Json& d : sh->items) {
      if (d.kind != Json::kNumber || !d.integral || d.inum < 0) fail("tensor '" + raw_name + "': bad dimension");
      e.shape.push_back(d.inum);
      if (d.inum != 0 && count > (std::uint64_t{1} << 62) / static_cast<std::uint64_t>(d.inum)) fail("tensor '" + raw_name + "': size overflows");
      count *= static_cast<std::uint64_t>(d.inum);
    }
    const Json &b = off->items[0], &en = off->items[1];
    if (b.kind != Json::kNumber || !b.integral || en.kind != Json::kNumber || !en.integral || b.inum < 0 || en.inum < b.inum ||
        static_cast<std::uint64_t>(en.inum) > data_bytes) {
      fail("tensor '" + raw_name + "': data_offsets outside the file");
    }
    e.offset = data_start + static_cast<std::uint64_t>(b.inum);
    e.nbytes = static_cast<std::uint64_t>(en.inum - b.inum);
    if (e.nbytes != count * esize) fail("tensor '" + raw_name + "': " + std::to_string(e.nbytes) + " bytes for " + e.describe());
    const std::string name = canonical(raw_name);
    if (!f->tensors.emplace(name, std::move(e)).second) fail("tensor '" + name + "' appears twice");
  }
}

// ------------------------------------------------------------------------------------------------ configs

struct Config {
  std::string format;
  bool convrot = false;
  std::int64_t convrot_groupsize = 256, group_size = 16, quant_group_size = 0;
  std::string linear_dtype;
};

Config parse_config(const Json& conf, const std::string& module) {
  if (conf.kind != Json::kObject) fail("quantization config of '" + module + "' is not a JSON object");
  const Json* f = conf.find("format");
  if (f == nullptr || f->kind != Json::kString) fail("quantization config of '" + module + "' has no format");
  Config c;
  c.format = f->str;
  // A field of the config or, as ComfyUI also accepts, of its "params" object.
  const auto field = [&](const char* key) -> const Json* {
    if (const Json* v = conf.find(key)) return v;
    const Json* p = conf.find("params");
    return p != nullptr && p->kind == Json::kObject ? p->find(key) : nullptr;
  };
  const auto get_int = [&](const char* key, std::int64_t& out) {
    if (const Json* v = field(key)) {
      if (v->kind != Json::kNumber || !v->integral) fail("'" + module + "': config field " + key + " is not an integer");
      out = v->inum;
    }
  };
  if (const Json* v = field("convrot")) {
    if (v->kind != Json::kBool) fail("'" + module + "': config field convrot is not a boolean");
    c.convrot = v->b;
  }
  get_int("convrot_groupsize", c.convrot_groupsize);
  get_int("group_size", c.group_size);
  get_int("quant_group_size", c.quant_group_size);
  if (const Json* v = field("linear_dtype")) {
    if (v->kind != Json::kString) fail("'" + module + "': config field linear_dtype is not a string");
    c.linear_dtype = v->str;
  }
  if (const Json* v = field("full_precision_matrix_mult"); v != nullptr && v->kind == Json::kBool && v->b) {
    fail("'" + module + "': full_precision_matrix_mult is not honoured");
  }
  return c;
}

std::map<std::string, Config> read_configs(const File& f) {
  std::map<std::string, Config> out;
  if (const auto it = f.metadata.find("_quantization_metadata"); it != f.metadata.end()) {
    const Json root = JsonParser(it->second.data(), it->second.size()).parse();
    const Json* layers = root.kind == Json::kObject ? root.find("layers") : nullptr;
    if (layers == nullptr || layers->kind != Json::kObject) fail("_quantization_metadata has no \"layers\" object");
    for (const auto& [module, conf] : layers->fields) out[canonical(module)] = parse_config(conf, module);
  }
  const std::string suffix = ".comfy_quant";
  for (const auto& [name, e] : f.tensors) {
    if (name.size() <= suffix.size() || name.compare(name.size() - suffix.size(), suffix.size(), suffix) != 0) continue;
    if (e.dtype != DT::kU8 || e.shape.size() != 1 || e.nbytes < 2 || e.nbytes > kMaxConfigBytes) {
      fail("'" + name + "' must be a U8 vector of 2.." + std::to_string(kMaxConfigBytes) + " bytes");
    }
    std::string text(static_cast<std::size_t>(e.nbytes), '\0');
    f.read(e.offset, text.data(), text.size());
    const std::string module = name.substr(0, name.size() - suffix.size());
    out[module] = parse_config(JsonParser(text.data(), text.size()).parse(), module);
  }
  return out;
}

// ------------------------------------------------------------------------------------------------ the model

enum class Enc { kInt8Rows, kInt8Scalar, kW4A4, kW4A8 };

// One stored linear, already checked against the shape the model gives it.
struct Stored {
  std::string module;
  Enc enc = Enc::kInt8Rows;
  std::int64_t n = 0, k = 0;
  int group = 0;  // W4A8 code group
  const Entry *weight = nullptr, *scale = nullptr, *s_rel = nullptr, *s_channel = nullptr, *codebook = nullptr;
};

bool per_row(const Entry& e, std::int64_t n) {
  return e.dtype == DT::kF32 && ((e.shape.size() == 1 && e.shape[0] == n) || (e.shape.size() == 2 && e.shape[0] == n && e.shape[1] == 1));
}

// The per-row scales of a stored linear (its only floats that steer the arithmetic), read and checked finite and > 0
// (quant_model.cpp:851) while the file is still only being described.
void check_scales(const File& f, const Stored& l) {
  const Entry& e = l.enc == Enc::kW4A8 ? *l.s_channel : *l.scale;
  std::vector<float> v(static_cast<std::size_t>(e.numel()));
  f.read(e.offset, v.data(), v.size() * 4);
  for (float s : v) {
    if (!(std::isfinite(s) && s > 0.0f)) fail("'" + l.module + "': a scale is not finite and > 0");
  }
  if (l.codebook != nullptr) {
    float cb[16];
    f.read(l.codebook->offset, cb, sizeof cb);
    for (float c : cb) {
      if (!std::isfinite(c)) fail("'" + l.module + "': non-finite codebook entry");
    }
  }
}

Stored stored_linear(const File& f, const std::map<std::string, Config>& configs, const std::string& m, std::int64_t n, std::int64_t k) {
  const auto cit = configs.find(m);
  if (cit == configs.end()) fail("'" + m + "' has no quantization config: the quantized block path needs every block linear quantized");
  const Config& c = cit->second;
  const auto take = [&](const std::string& name) {
    const Entry* e = f.find(name);
    if (e == nullptr) fail("tensor '" + name + "' missing");
    return e;
  };
  Stored l;
  l.module = m;
  l.weight = take(m + ".weight");
  if (f.find(m + ".bias") != nullptr) fail("'" + m + "' has a bias the DiT does not use");
  if (c.format == "w6a8_int8" || c.format == "nvfp4") fail("'" + m + "': format " + c.format + " is not read by this library");
  if (c.format != "int8_tensorwise" && c.format != "convrot_w4a4" && c.format != "asym_w4a8_int8") {
    fail("'" + m + "': quantization format '" + c.format + "' is not supported");
  }
  const Entry& w = *l.weight;
  if (w.dtype != DT::kI8 || w.shape.size() != 2 || w.shape[0] <= 0 || w.shape[1] <= 0) {
    fail("'" + m + "': " + c.format + " weight must be I8 [N, C], got " + w.describe());
  }
  l.n = w.shape[0];
  const std::int64_t cols = w.shape[1];
  const auto need_rotation = [&] {
    if (c.convrot_groupsize != 256) fail("'" + m + "': rotation group " + std::to_string(c.convrot_groupsize) + ", the kernels rotate by 256");
  };
  if (c.format == "int8_tensorwise") {
    if (!c.convrot) fail("'" + m + "': plain INT8 without rotation does not fit the block, whose activations are rotated");
    need_rotation();
    l.k = cols;
    l.scale = take(m + ".weight_scale");
    if (per_row(*l.scale, l.n)) l.enc = Enc::kInt8Rows;
    else if (l.scale->dtype == DT::kF32 && l.scale->numel() == 1) l.enc = Enc::kInt8Scalar;
    else fail("'" + m + "': weight_scale must be F32 [N], [N, 1] or a scalar, got " + l.scale->describe());
  } else if (c.format == "convrot_w4a4") {
    need_rotation();
    l.k = cols * 2;
    l.enc = Enc::kW4A4;
    if (c.quant_group_size != 0 && l.k % c.quant_group_size != 0) fail("'" + m + "': quant_group_size does not divide K");
    if (!c.linear_dtype.empty() && c.linear_dtype != "int4" && c.linear_dtype != "int8") fail("'" + m + "': unknown linear_dtype '" + c.linear_dtype + "'");
    l.scale = take(m + ".weight_scale");
    if (!per_row(*l.scale, l.n)) fail("'" + m + "': convrot_w4a4 weight_scale must be F32 [N]");
  } else {
    need_rotation();
    l.k = cols * 2;
    l.enc = Enc::kW4A8;
    const std::int64_t gs = c.group_size;
    if (gs < 16 || gs % 16 != 0 || l.k % 16 != 0 || l.k % gs != 0) {
      fail("'" + m + "': group_size " + std::to_string(gs) + " / K=" + std::to_string(l.k) + ": this library decodes groups that are multiples of 16");
    }
    l.group = static_cast<int>(gs);
    l.s_rel = take(m + ".weight_s_rel");
    if ((l.s_rel->dtype != DT::kF8E4M3 && l.s_rel->dtype != DT::kU8) || l.s_rel->shape != std::vector<std::int64_t>{l.n, l.k / gs}) {
      fail("'" + m + "': weight_s_rel must be F8_E4M3 [" + std::to_string(l.n) + ", " + std::to_string(l.k / gs) + "], got " + l.s_rel->describe());
    }
    l.s_channel = take(m + ".weight_s_channel");
    if (!per_row(*l.s_channel, l.n)) fail("'" + m + "': weight_s_channel must be F32 [N]");
    l.codebook = f.find(m + ".weight_codebook");
    if (l.codebook != nullptr && (l.codebook->dtype != DT::kF32 || l.codebook->shape != std::vector<std::int64_t>{16})) {
      fail("'" + m + "': weight_codebook must be F32 [16]");
    }
  }
  if (l.n != n || l.k != k) {
    fail("'" + m + "' is [" + std::to_string(l.n) + ", " + std::to_string(l.k) + "], the DiT's is [" + std::to_string(n) + ", " + std::to_string(k) + "]");
  }
  check_scales(f, l);
  return l;
}

int tier_of(Enc e) { return e == Enc::kW4A4 ? B2_TIER_W4A4_VIA_INT8 : e == Enc::kW4A8 ? B2_TIER_W4A8 : B2_TIER_INT8; }

// Device memory of the loaded model: one allocation, carved in 256-byte steps.
struct Arena {
  unsigned char* base = nullptr;
  std::size_t size = 0, used = 0;
  ~Arena() {
    if (base != nullptr) cudaFree(base);
  }
  void* take(std::size_t bytes) {
    const std::size_t at = used;
    used += (bytes + 255) & ~std::size_t{255};
    if (used > size) fail("internal: device arena too small");
    return base + at;
  }
};

std::size_t padded(std::uint64_t bytes) { return static_cast<std::size_t>((bytes + 255) & ~std::uint64_t{255}); }

}  // namespace
}  // namespace b2

using namespace b2;

struct b2_dit_file {
  Arena arena;
  std::vector<b2_block_weights> blocks;
  std::vector<std::unique_ptr<b2_w4_weight>> w4;  // stable addresses for b2_linear::w4
  b2_dit_model model{};
  b2_time_embedding time{};
  b2_time_mlp_bf16 time_bf16{};  // the same MLP and the modulation linears as bf16 device tensors (struct_size 0: absent)
  std::vector<float> te_w0, te_b0, te_w2, te_b2;
  b2_dit_file_info info{};
};

namespace b2 {
namespace {

// Two pinned host buffers and a copy stream: the file read of one chunk overlaps the device copy of the one before.
struct Staging {
  static constexpr std::size_t kChunk = std::size_t{32} << 20;
  unsigned char* buf[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  cudaStream_t stream = nullptr;
  int next = 0;
  Staging() {
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) fail("cannot create a copy stream");
    for (int i = 0; i < 2; ++i) {
      if (cudaHostAlloc(reinterpret_cast<void**>(&buf[i]), kChunk, cudaHostAllocDefault) != cudaSuccess ||
          cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) != cudaSuccess) {
        fail("cannot allocate the pinned staging buffers");
      }
    }
  }
  ~Staging() {
    if (stream != nullptr) cudaStreamSynchronize(stream);
    for (int i = 0; i < 2; ++i) {
      if (done[i] != nullptr) cudaEventDestroy(done[i]);
      if (buf[i] != nullptr) cudaFreeHost(buf[i]);
    }
    if (stream != nullptr) cudaStreamDestroy(stream);
  }
  void drain() {
    if (const cudaError_t err = cudaStreamSynchronize(stream); err != cudaSuccess) fail(std::string("copy to the device failed: ") + cudaGetErrorString(err));
  }
};

struct Loader {
  const File& f;
  b2_dit_file& out;
  bool expand = false;  // grouped 4-bit weights (W4A8) are expanded to the INT8 grid once, here, and the blocks run the INT8 tier
  Staging staging;

  // Tensor bytes -> device, in chunks through the pinned buffers.
  void upload(const Entry& e, void* dst, std::uint64_t first = 0, std::uint64_t bytes = ~std::uint64_t{0}) {
    if (bytes == ~std::uint64_t{0}) bytes = e.nbytes - first;
    for (std::uint64_t at = 0; at < bytes; at += Staging::kChunk) {
      const std::size_t n = static_cast<std::size_t>(std::min<std::uint64_t>(Staging::kChunk, bytes - at));
      const int b = staging.next;
      staging.next ^= 1;
      cudaEventSynchronize(staging.done[b]);  // the copy that last used this buffer
      f.read(e.offset + first + at, staging.buf[b], n);
      cudaError_t err = cudaMemcpyAsync(static_cast<unsigned char*>(dst) + at, staging.buf[b], n, cudaMemcpyHostToDevice, staging.stream);
      if (err == cudaSuccess) err = cudaEventRecord(staging.done[b], staging.stream);
      if (err != cudaSuccess) fail(std::string("copy to the device failed: ") + cudaGetErrorString(err));
    }
  }
  std::vector<float> floats(const Entry& e) {
    std::vector<float> v(static_cast<std::size_t>(e.numel()));
    if (e.dtype == DT::kF32) {
      f.read(e.offset, v.data(), v.size() * 4);
    } else if (e.dtype == DT::kBF16) {
      std::vector<std::uint16_t> raw(v.size());
      f.read(e.offset, raw.data(), raw.size() * 2);
      for (std::size_t i = 0; i < v.size(); ++i) {
        const std::uint32_t bits = static_cast<std::uint32_t>(raw[i]) << 16;
        std::memcpy(&v[i], &bits, 4);
      }
    } else {
      fail("expected F32 or BF16, got " + e.describe());
    }
    return v;
  }
  // Per-row scales of a linear, checked finite and > 0 (quant_model.cpp:851), n floats on the device.
  void upload_scales(const Stored& l, const Entry& e, float* dst, bool scalar) {
    std::vector<float> v = floats(e);
    if (scalar) v.assign(static_cast<std::size_t>(l.n), v.at(0));
    for (float s : v) {
      if (!(std::isfinite(s) && s > 0.0f)) fail("'" + l.module + "': a scale is not finite and > 0");
    }
    if (const cudaError_t err = cudaMemcpy(dst, v.data(), v.size() * 4, cudaMemcpyHostToDevice); err != cudaSuccess) {
      fail(std::string("copy to the device failed: ") + cudaGetErrorString(err));
    }
  }
  // A bf16 device vector or matrix from a BF16 or F32 tensor.
  const void* upload_bf16(const std::string& name, std::vector<std::int64_t> shape) {
    const Entry* e = f.find(name);
    if (e == nullptr) fail("tensor '" + name + "' missing");
    if (e->shape != shape || (e->dtype != DT::kBF16 && e->dtype != DT::kF32)) fail("'" + name + "' must be BF16 (or F32) of the model's shape, got " + e->describe());
    void* dst = out.arena.take(static_cast<std::size_t>(e->numel()) * 2);
    if (e->dtype == DT::kBF16) {
      upload(*e, dst);
    } else {
      const std::vector<float> v = floats(*e);
      std::vector<std::uint16_t> h(v.size());
      for (std::size_t i = 0; i < v.size(); ++i) {
        std::uint32_t u;
        std::memcpy(&u, &v[i], 4);
        h[i] = std::isnan(v[i]) ? 0x7FFF : static_cast<std::uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
      }
      cudaMemcpy(dst, h.data(), h.size() * 2, cudaMemcpyHostToDevice);
    }
    return dst;
  }
  const float* upload_f32(const std::string& name, std::int64_t n) {
    const Entry* e = f.find(name);
    if (e == nullptr) fail("tensor '" + name + "' missing");
    if (e->numel() != n || e->shape.size() != 1) fail("'" + name + "' must hold " + std::to_string(n) + " values, got " + e->describe());
    const std::vector<float> v = floats(*e);
    float* dst = static_cast<float*>(out.arena.take(v.size() * 4));
    cudaMemcpy(dst, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return dst;
  }

  // One linear of a block from its parts (three for q | k | v, else one), stacked by rows.
  b2_linear linear(const std::vector<Stored>& parts) {
    const Stored& a = parts.front();
    std::int64_t n = 0;
    for (const Stored& p : parts) n += p.n;
    b2_linear lin{};
    if (a.enc == Enc::kW4A8) {
      auto w4 = std::make_unique<b2_w4_weight>();
      unsigned char* packed = static_cast<unsigned char*>(out.arena.take(static_cast<std::size_t>(n * a.k / 2)));
      unsigned char* s_rel = static_cast<unsigned char*>(out.arena.take(static_cast<std::size_t>(n * a.k / a.group)));
      float* s_channel = static_cast<float*>(out.arena.take(static_cast<std::size_t>(n) * 4));
      std::int64_t row = 0;
      for (const Stored& p : parts) {
        upload(*p.weight, packed + row * a.k / 2);
        upload(*p.s_rel, s_rel + row * a.k / a.group);
        upload_scales(p, *p.s_channel, s_channel + row, false);
        row += p.n;
      }
      w4->packed = packed, w4->s_rel = s_rel, w4->scale_kind = 0, w4->group = a.group, w4->s_channel = s_channel;
      if (a.codebook != nullptr) {
        const std::vector<float> cb = floats(*a.codebook);
        for (float v : cb) {
          if (!std::isfinite(v)) fail("'" + a.module + "': non-finite codebook entry");
        }
        for (const Stored& p : parts) {
          if (p.codebook == nullptr || floats(*p.codebook) != cb) fail("'" + a.module + "': q, k and v need one codebook to run as one GEMM");
        }
        float* dst = static_cast<float*>(out.arena.take(64));
        cudaMemcpy(dst, cb.data(), 64, cudaMemcpyHostToDevice);
        w4->codebook = dst;
      } else {
        for (const Stored& p : parts) {
          if (p.codebook != nullptr) fail("'" + a.module + "': q, k and v need one codebook to run as one GEMM");
        }
      }
      if (expand) {
        // quant::decode_grouped_int8 on the copy stream, behind the uploads it reads: the INT8 GEMM over these values with
        // s_channel as the weight scale is what the W4A8 tier computes on every step.
        std::int8_t* dec = static_cast<std::int8_t*>(out.arena.take(static_cast<std::size_t>(n * a.k)));
        if (b2_decode_grouped_int8(packed, s_rel, 0, w4->codebook, n, a.k, a.group, dec, nullptr, staging.stream) != B2_OK) {
          fail("'" + a.module + "': " + b2_last_error_message());
        }
        lin.w = dec, lin.scale = s_channel;
        return lin;
      }
      lin.w4 = w4.get();
      out.w4.push_back(std::move(w4));
      return lin;
    }
    const std::int64_t row_bytes = a.enc == Enc::kW4A4 ? a.k / 2 : a.k;
    unsigned char* w = static_cast<unsigned char*>(out.arena.take(static_cast<std::size_t>(n * row_bytes)));
    float* s = static_cast<float*>(out.arena.take(static_cast<std::size_t>(n) * 4));
    std::int64_t row = 0;
    for (const Stored& p : parts) {
      upload(*p.weight, w + row * row_bytes);
      upload_scales(p, *p.scale, s + row, p.enc == Enc::kInt8Scalar);
      row += p.n;
    }
    lin.w = reinterpret_cast<const std::int8_t*>(w), lin.scale = s;
    return lin;
  }
};

std::size_t linear_bytes(const std::vector<Stored>& parts, bool expand) {
  std::size_t total = 0;
  for (const Stored& p : parts) {
    total += padded(p.weight->nbytes) + padded(static_cast<std::uint64_t>(p.n) * 4) + 512;
    if (p.s_rel != nullptr) total += padded(p.s_rel->nbytes) + 512;
    if (expand && p.enc == Enc::kW4A8) total += padded(static_cast<std::uint64_t>(p.n) * static_cast<std::uint64_t>(p.k)) + 512;
  }
  return total + 1024;
}

}  // namespace
}  // namespace b2

namespace b2 {
namespace {
int open_impl(const char* op, const char* path, bool expand, b2_dit_file** out) {
  if (path == nullptr || out == nullptr) return fail_invalid(op, "null argument");
  *out = nullptr;
  try {
    File f;
    open_file(path, &f);
    const std::map<std::string, Config> configs = read_configs(f);
    // Blocks 0 .. B-1, contiguous.
    int blocks = 0;
    while (f.find("layers." + std::to_string(blocks) + ".norm1.weight") != nullptr) ++blocks;
    if (blocks == 0) fail("no 'layers.0.norm1.weight': not a MOSS-Image DiT file");
    if (blocks > 64) fail("more than 64 blocks");
    const Entry* down0 = f.find("layers.0.proj.ffn_down.weight");
    const auto cfg0 = configs.find("layers.0.proj.ffn_down");
    if (down0 == nullptr || down0->shape.size() != 2 || cfg0 == configs.end()) fail("'layers.0.proj.ffn_down' missing or without a quantization config");
    const std::int64_t F = cfg0->second.format == "int8_tensorwise" ? down0->shape[1] : down0->shape[1] * 2;
    if (F <= 0 || F % 256 != 0 || F > 32768) fail("FFN width " + std::to_string(F) + " is not a multiple of 256 up to 32768");

    // Describe and check everything before reading a tensor byte.
    std::vector<std::vector<std::vector<Stored>>> plan(static_cast<std::size_t>(blocks));  // [block][qkv, o, up_gate, down][parts]
    int tier = -1;
    std::size_t need = 4096;
    for (int b = 0; b < blocks; ++b) {
      const std::string p = "layers." + std::to_string(b) + ".";
      for (const auto& [name, len] : {std::pair<const char*, std::int64_t>{"norm1.weight", kDim}, {"norm2.weight", kDim}, {"q_norm.weight", kHeadDim}, {"k_norm.weight", kHeadDim}}) {
        const Entry* e = f.find(p + name);
        if (e == nullptr || e->shape != std::vector<std::int64_t>{len} || (e->dtype != DT::kBF16 && e->dtype != DT::kF32)) {
          fail("'" + p + name + "' must be BF16 [" + std::to_string(len) + "]" + (e != nullptr ? ", got " + e->describe() : " and is missing"));
        }
        need += padded(static_cast<std::uint64_t>(len) * 2);
      }
      std::vector<Stored> qkv;
      if (f.find(p + "proj.qkv.weight") != nullptr) {
        qkv.push_back(stored_linear(f, configs, p + "proj.qkv", 3 * kDim, kDim));
      } else {
        for (const char* part : {"proj.q", "proj.k", "proj.v"}) qkv.push_back(stored_linear(f, configs, p + part, kDim, kDim));
        for (const Stored& s : qkv) {
          if (tier_of(s.enc) != tier_of(qkv[0].enc) || s.group != qkv[0].group) fail("'" + p + "proj.q/k/v' are stored in different formats: one fused GEMM needs one");
        }
      }
      plan[static_cast<std::size_t>(b)] = {qkv, {stored_linear(f, configs, p + "proj.o", kDim, kDim)},
                                           {stored_linear(f, configs, p + "proj.ffn_up_gate", 2 * F, kDim)},
                                           {stored_linear(f, configs, p + "proj.ffn_down", kDim, F)}};
      for (const auto& parts : plan[static_cast<std::size_t>(b)]) {
        const int t = tier_of(parts[0].enc);
        if (tier >= 0 && t != tier) fail("'" + parts[0].module + "' is of another tier than the linears before it: a block run has one tier");
        tier = t;
        need += linear_bytes(parts, expand);
      }
    }
    const bool shell = f.find("shared_block_modulation.weight") != nullptr;
    const bool has_time = f.find("time_embedding.0.weight") != nullptr;
    if (shell) need += padded(6 * kDim * kDim * 2) + padded(2 * kDim * kDim * 2) + padded(kDim * kLatent * 2) * 2 + padded(8 * kDim * 4) + padded(kDim * 2) * 3 + 8192;
    // The bf16 form of the time modulation: the timestep MLP and bf16 copies of the two modulation biases.
    if (shell && has_time) need += padded(kDim * kFreq * 2) + padded(kDim * kDim * 2) + padded(kDim * 2) * 2 + padded(8 * kDim * 2) + 4096;

    auto file = std::make_unique<b2_dit_file>();
    if (const cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&file->arena.base), need); err != cudaSuccess) {
      return fail_cuda(op, err);
    }
    file->arena.size = need;
    Loader ld{f, *file, expand};
    file->blocks.resize(static_cast<std::size_t>(blocks));
    for (int b = 0; b < blocks; ++b) {
      const std::string p = "layers." + std::to_string(b) + ".";
      b2_block_weights& w = file->blocks[static_cast<std::size_t>(b)];
      w.struct_size = sizeof w;
      w.norm1 = ld.upload_bf16(p + "norm1.weight", {kDim});
      w.norm2 = ld.upload_bf16(p + "norm2.weight", {kDim});
      w.q_norm = ld.upload_bf16(p + "q_norm.weight", {kHeadDim});
      w.k_norm = ld.upload_bf16(p + "k_norm.weight", {kHeadDim});
      const auto& lp = plan[static_cast<std::size_t>(b)];
      w.qkv = ld.linear(lp[0]), w.o = ld.linear(lp[1]), w.up_gate = ld.linear(lp[2]), w.down = ld.linear(lp[3]);
    }
    b2_dit_model& m = file->model;
    m.struct_size = sizeof m;
    m.blocks = file->blocks.data(), m.num_blocks = blocks, m.D = static_cast<int>(kDim), m.F = static_cast<int>(F), m.heads = 24;
    m.latent_channels = static_cast<int>(kLatent);
    if (shell) {
      m.block_mod_w = ld.upload_bf16("shared_block_modulation.weight", {6 * kDim, kDim});
      m.block_mod_bias = ld.upload_f32("shared_block_modulation.bias", 6 * kDim);
      m.head_mod_w = ld.upload_bf16("video_head_modulation.weight", {2 * kDim, kDim});
      m.head_mod_bias = ld.upload_f32("video_head_modulation.bias", 2 * kDim);
      m.video_w = ld.upload_bf16("video_embedder.weight", {kDim, kLatent});
      m.video_bias = ld.upload_bf16("video_embedder.bias", {kDim});
      m.final_norm = ld.upload_bf16("final_norm_video.weight", {kDim});
      m.final_w = ld.upload_bf16("final_linear_video.weight", {kLatent, kDim});
    }
    if (has_time) {
      const auto host = [&](const std::string& name, std::vector<std::int64_t> shape) {
        const Entry* e = f.find(name);
        if (e == nullptr || e->shape != shape) fail("'" + name + "' missing or of an unexpected shape");
        return ld.floats(*e);
      };
      file->te_w0 = host("time_embedding.0.weight", {kDim, kFreq});
      file->te_b0 = host("time_embedding.0.bias", {kDim});
      file->te_w2 = host("time_embedding.2.weight", {kDim, kDim});
      file->te_b2 = host("time_embedding.2.bias", {kDim});
      file->time = b2_time_embedding{sizeof(b2_time_embedding), kDim, file->te_w0.data(), file->te_b0.data(), file->te_w2.data(), file->te_b2.data()};
      if (shell) {
        b2_time_mlp_bf16& t = file->time_bf16;
        t.dim = kDim;
        t.in_w = ld.upload_bf16("time_embedding.0.weight", {kDim, kFreq});
        t.in_bias = ld.upload_bf16("time_embedding.0.bias", {kDim});
        t.out_w = ld.upload_bf16("time_embedding.2.weight", {kDim, kDim});
        t.out_bias = ld.upload_bf16("time_embedding.2.bias", {kDim});
        t.block_mod_w = m.block_mod_w;
        t.block_mod_bias = ld.upload_bf16("shared_block_modulation.bias", {6 * kDim});
        t.head_mod_w = m.head_mod_w;
        t.head_mod_bias = ld.upload_bf16("video_head_modulation.bias", {2 * kDim});
        t.struct_size = sizeof(b2_time_mlp_bf16);
      }
    }
    ld.staging.drain();
    file->info = b2_dit_file_info{sizeof(b2_dit_file_info), blocks, static_cast<int>(F), expand && tier == B2_TIER_W4A8 ? B2_TIER_INT8 : tier, shell ? 1 : 0, has_time ? 1 : 0, file->arena.used, tier};
    *out = file.release();
    return B2_OK;
  } catch (const LoadError& e) {
    return fail_invalid(op, std::string(path) + ": " + e.what);
  } catch (const std::bad_alloc&) {
    return fail_status(B2_ERR_INTERNAL, op, "out of host memory");
  } catch (const std::exception& e) {  // nothing may cross the C boundary
    return fail_status(B2_ERR_INTERNAL, op, std::string(path) + ": " + e.what());
  }
}

}  // namespace
}  // namespace b2

extern "C" {

int b2_dit_file_open(const char* path, b2_dit_file** out) { return open_impl("dit_file_open", path, false, out); }

int b2_dit_file_open_expanded(const char* path, b2_dit_file** out) { return open_impl("dit_file_open_expanded", path, true, out); }

int b2_dit_file_get_info(const b2_dit_file* file, b2_dit_file_info* info) {
  constexpr std::size_t kFirst = offsetof(b2_dit_file_info, stored_tier);  // the struct before stored_tier was added
  if (file == nullptr || info == nullptr || info->struct_size < kFirst) return fail_invalid("dit_file_get_info", "null argument or an older header");
  const std::size_t theirs = info->struct_size;
  std::memcpy(info, &file->info, std::min(theirs, sizeof(b2_dit_file_info)));
  info->struct_size = theirs;
  return B2_OK;
}

const b2_dit_model* b2_dit_file_model(const b2_dit_file* file) { return file == nullptr ? nullptr : &file->model; }

const b2_time_embedding* b2_dit_file_time_embedding(const b2_dit_file* file) {
  return file == nullptr || file->info.has_time_embedding == 0 ? nullptr : &file->time;
}

const b2_time_mlp_bf16* b2_dit_file_time_mlp_bf16(const b2_dit_file* file) {
  return file == nullptr || file->time_bf16.struct_size == 0 ? nullptr : &file->time_bf16;
}

void b2_dit_file_close(b2_dit_file* file) { delete file; }

}  // extern "C"
