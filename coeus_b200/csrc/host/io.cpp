#include "io.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <stdexcept>

namespace coeus {

// ------------------------------------------------------------------------------ mmap
MappedFile::MappedFile(const std::string& path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) throw std::runtime_error("io: cannot open '" + path + "'");
  struct stat st;
  if (fstat(fd_, &st) != 0) { ::close(fd_); throw std::runtime_error("io: fstat failed"); }
  size_ = static_cast<size_t>(st.st_size);
  if (size_ > 0) {
    void* p = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (p == MAP_FAILED) { ::close(fd_); throw std::runtime_error("io: mmap failed"); }
    data_ = static_cast<uint8_t*>(p);
  }
}
MappedFile::~MappedFile() {
  if (data_) ::munmap(data_, size_);
  if (fd_ >= 0) ::close(fd_);
}

// ------------------------------------------------------------------------------ little endian
template <typename T>
static void put_le(std::string& out, T v) {
  for (size_t i = 0; i < sizeof(T); ++i) out.push_back(static_cast<char>((v >> (8 * i)) & 0xFF));
}
template <typename T>
static T get_le(const uint8_t* p) {
  T v = 0;
  for (size_t i = 0; i < sizeof(T); ++i) v |= static_cast<T>(p[i]) << (8 * i);
  return v;
}

// ------------------------------------------------------------------------------ .rustllm
uint64_t rustllm_checksum(const float* p, size_t n, uint64_t c) {
  for (size_t i = 0; i < n; ++i) {
    uint32_t bits;
    std::memcpy(&bits, p + i, 4);
    c += bits;
    c = (c << 1) | (c >> 63);
  }
  return c;
}

std::string rustllm_pack_header(const RustllmHeader& h) {
  std::string out;
  out.append("RUSTLLM", 7);
  out.push_back('\0');
  put_le<uint32_t>(out, h.format_version);
  put_le<uint16_t>(out, h.ver_major);
  put_le<uint16_t>(out, h.ver_minor);
  put_le<uint16_t>(out, h.ver_patch);
  out.append(6, '\0');  // struct padding (uninitialised in the reference; zero here)
  put_le<uint64_t>(out, h.param_count);
  put_le<uint64_t>(out, h.param_bytes);
  put_le<uint64_t>(out, h.param_offset);
  put_le<uint64_t>(out, h.metadata_offset);
  put_le<uint64_t>(out, h.metadata_size);
  put_le<uint64_t>(out, h.checksum);
  out.append(64, '\0');  // reserved [u64; 8]
  return out;
}

RustllmHeader rustllm_unpack_header(const uint8_t* b, size_t n) {
  if (n < kRustllmHeaderBytes) throw std::invalid_argument("Invalid magic bytes");
  if (std::memcmp(b, "RUSTLLM\0", 8) != 0) throw std::invalid_argument("Invalid magic bytes");
  RustllmHeader h;
  h.format_version = get_le<uint32_t>(b + 8);
  if (h.format_version != 1)
    throw std::invalid_argument("Unsupported format version: " + std::to_string(h.format_version));
  h.ver_major = get_le<uint16_t>(b + 12);
  h.ver_minor = get_le<uint16_t>(b + 14);
  h.ver_patch = get_le<uint16_t>(b + 16);
  h.param_count = get_le<uint64_t>(b + 24);
  h.param_bytes = get_le<uint64_t>(b + 32);
  h.param_offset = get_le<uint64_t>(b + 40);
  h.metadata_offset = get_le<uint64_t>(b + 48);
  h.metadata_size = get_le<uint64_t>(b + 56);
  h.checksum = get_le<uint64_t>(b + 64);
  return h;
}

static void put_lp(std::string& out, const std::string& s) {
  put_le<uint32_t>(out, static_cast<uint32_t>(s.size()));
  out += s;
}

std::string rustllm_metadata_to_bytes(const RustllmMetadata& m) {
  std::string out;
  put_lp(out, m.architecture);
  if (m.has_training_config) {
    out.push_back(1);
    put_lp(out, m.training_config);
  } else {
    out.push_back(0);
  }
  put_le<uint32_t>(out, static_cast<uint32_t>(m.custom.size()));
  for (auto& kv : m.custom) {
    put_lp(out, kv.first);
    put_lp(out, kv.second);
  }
  return out;
}

static bool valid_utf8(const std::string& s) {
  size_t i = 0;
  while (i < s.size()) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    size_t len = c < 0x80 ? 1 : (c & 0xE0) == 0xC0 ? 2 : (c & 0xF0) == 0xE0 ? 3 : (c & 0xF8) == 0xF0 ? 4 : 0;
    if (len == 0 || i + len > s.size()) return false;
    for (size_t k = 1; k < len; ++k)
      if ((static_cast<unsigned char>(s[i + k]) & 0xC0) != 0x80) return false;
    i += len;
  }
  return true;
}

RustllmMetadata rustllm_metadata_from_bytes(const uint8_t* b, size_t n) {
  size_t cur = 0;
  auto need = [&](size_t k) {
    if (n < cur + k) throw std::invalid_argument("Invalid metadata format");
  };
  auto read_str = [&]() {
    need(4);
    const uint32_t len = get_le<uint32_t>(b + cur);
    cur += 4;
    need(len);
    std::string s(reinterpret_cast<const char*>(b + cur), len);
    cur += len;
    if (!valid_utf8(s)) throw std::invalid_argument("Invalid UTF-8 in metadata");
    return s;
  };
  RustllmMetadata m;
  m.architecture = read_str();
  need(1);
  m.has_training_config = b[cur++] != 0;
  if (m.has_training_config) m.training_config = read_str();
  need(4);
  const uint32_t count = get_le<uint32_t>(b + cur);
  cur += 4;
  for (uint32_t i = 0; i < count; ++i) {
    std::string k = read_str();
    std::string v = read_str();
    m.custom.emplace_back(std::move(k), std::move(v));
  }
  return m;
}

RustllmHeader rustllm_write(const std::string& path, const float* params, size_t n,
                            const RustllmMetadata& meta, const Progress& progress) {
  RustllmHeader h;
  h.param_count = n;
  h.param_bytes = 4ull * n;
  h.param_offset = kRustllmHeaderBytes;
  h.metadata_offset = kRustllmHeaderBytes + 4ull * n;
  const std::string mbytes = rustllm_metadata_to_bytes(meta);
  h.metadata_size = mbytes.size();
  FILE* f = std::fopen(path.c_str(), "wb");
  if (!f) throw std::runtime_error("io failed: cannot create '" + path + "'");
  const std::string placeholder = rustllm_pack_header(h);
  std::fwrite(placeholder.data(), 1, placeholder.size(), f);
  // 8 MiB chunks; x86-64 / aarch64 are little endian, so fp32 goes out as it lies in memory.
  // The checksum is sequential by definition and is folded into the same pass.
  const size_t chunk = (8u << 20) / 4;
  uint64_t cks = 0;
  size_t done = 0;
  while (done < n) {
    const size_t k = std::min(chunk, n - done);
    cks = rustllm_checksum(params + done, k, cks);
    if (std::fwrite(params + done, 4, k, f) != k) {
      std::fclose(f);
      throw std::runtime_error("io failed: Failed to write parameters");
    }
    done += k;
    if (progress) progress(done * 4, n * 4);
  }
  std::fwrite(mbytes.data(), 1, mbytes.size(), f);
  h.checksum = cks;
  const std::string header = rustllm_pack_header(h);
  std::fseek(f, 0, SEEK_SET);
  std::fwrite(header.data(), 1, header.size(), f);
  std::fclose(f);
  return h;
}

RustllmHeader rustllm_read(const std::string& path, std::vector<float>& params,
                           RustllmMetadata& meta, const Progress& progress) {
  MappedFile mf(path);
  RustllmHeader h = rustllm_unpack_header(mf.data(), mf.size());
  if (h.param_offset + 4 * h.param_count > mf.size())
    throw std::runtime_error("io failed: Failed to read parameters: file too short");
  params.resize(h.param_count);
  const size_t chunk = (8u << 20) / 4;
  uint64_t cks = 0;
  size_t done = 0;
  const uint8_t* src = mf.data() + h.param_offset;
  while (done < h.param_count) {
    const size_t k = std::min<size_t>(chunk, h.param_count - done);
    std::memcpy(params.data() + done, src + 4 * done, 4 * k);
    cks = rustllm_checksum(params.data() + done, k, cks);
    done += k;
    if (progress) progress(done * 4, h.param_count * 4);
  }
  if (cks != h.checksum) throw std::runtime_error("internal failed: Checksum mismatch");
  if (h.metadata_offset + h.metadata_size > mf.size())
    throw std::invalid_argument("Invalid metadata format");
  meta = rustllm_metadata_from_bytes(mf.data() + h.metadata_offset, h.metadata_size);
  return h;
}

// ------------------------------------------------------------------------------ dtypes
size_t dtype_size(const std::string& d) {
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "U8" || d == "I8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  throw std::invalid_argument("io: unknown dtype '" + d + "'");
}

// ------------------------------------------------------------------------------ JSON (subset)
static void json_escape(std::string& out, const std::string& s) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\u%04x", c);
          out += buf;
        } else {
          out.push_back(static_cast<char>(c));
        }
    }
  }
  out.push_back('"');
}

struct JsonCursor {
  const char* p;
  const char* end;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  void expect(char c) {
    ws();
    if (p >= end || *p != c) throw std::invalid_argument("safetensors: malformed JSON header");
    ++p;
  }
  bool peek(char c) { ws(); return p < end && *p == c; }
  std::string str() {
    expect('"');
    std::string out;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            if (p + 4 >= end) throw std::invalid_argument("safetensors: bad escape");
            unsigned cp = 0;
            for (int i = 1; i <= 4; ++i) {
              const char c = p[i];
              cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 0x20) - 'a' + 10);
            }
            p += 4;
            if (cp < 0x80) out.push_back(static_cast<char>(cp));
            else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
            else { out.push_back(static_cast<char>(0xE0 | (cp >> 12))); out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
            break;
          }
          default: out.push_back(*p);
        }
        ++p;
      } else {
        out.push_back(*p++);
      }
    }
    expect('"');
    return out;
  }
  uint64_t num() {
    ws();
    uint64_t v = 0;
    bool any = false;
    while (p < end && *p >= '0' && *p <= '9') { v = v * 10 + static_cast<uint64_t>(*p - '0'); ++p; any = true; }
    if (!any) throw std::invalid_argument("safetensors: expected a number");
    return v;
  }
  std::vector<uint64_t> num_array() {
    std::vector<uint64_t> out;
    expect('[');
    if (peek(']')) { ++p; return out; }
    while (true) {
      out.push_back(num());
      if (peek(',')) { ++p; continue; }
      expect(']');
      return out;
    }
  }
};

// ------------------------------------------------------------------------------ SafeTensors
void safetensors_write(const std::string& path, const std::vector<TensorToWrite>& tensors,
                       const std::map<std::string, std::string>& metadata) {
  std::string json = "{";
  if (!metadata.empty()) {
    json += "\"__metadata__\":{";
    bool first = true;
    for (auto& kv : metadata) {
      if (!first) json.push_back(',');
      first = false;
      json_escape(json, kv.first);
      json.push_back(':');
      json_escape(json, kv.second);
    }
    json += "}";
  }
  uint64_t off = 0;
  bool first = metadata.empty();
  for (auto& t : tensors) {
    if (!first) json.push_back(',');
    first = false;
    json_escape(json, t.name);
    json += ":{\"dtype\":\"" + t.dtype + "\",\"shape\":[";
    for (size_t i = 0; i < t.shape.size(); ++i) {
      if (i) json.push_back(',');
      json += std::to_string(t.shape[i]);
    }
    json += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + t.nbytes) + "]}";
    off += t.nbytes;
  }
  json += "}";
  while (json.size() % 8) json.push_back(' ');
  FILE* f = std::fopen(path.c_str(), "wb");
  if (!f) throw std::runtime_error("io failed: cannot create '" + path + "'");
  std::string len;
  put_le<uint64_t>(len, json.size());
  std::fwrite(len.data(), 1, 8, f);
  std::fwrite(json.data(), 1, json.size(), f);
  for (auto& t : tensors)
    if (t.nbytes && std::fwrite(t.data, 1, t.nbytes, f) != t.nbytes) {
      std::fclose(f);
      throw std::runtime_error("io failed: short write");
    }
  std::fclose(f);
}

TensorFile safetensors_index(const std::string& path) {
  MappedFile mf(path);
  if (mf.size() < 8) throw std::invalid_argument("safetensors: file too short");
  const uint64_t n = get_le<uint64_t>(mf.data());
  if (8 + n > mf.size()) throw std::invalid_argument("safetensors: header length out of range");
  JsonCursor c{reinterpret_cast<const char*>(mf.data() + 8), reinterpret_cast<const char*>(mf.data() + 8 + n)};
  TensorFile out;
  c.expect('{');
  if (c.peek('}')) return out;
  while (true) {
    const std::string key = c.str();
    c.expect(':');
    c.expect('{');
    if (key == "__metadata__") {
      if (!c.peek('}')) {
        while (true) {
          const std::string k = c.str();
          c.expect(':');
          out.metadata[k] = c.str();
          if (c.peek(',')) { ++c.p; continue; }
          break;
        }
      }
      c.expect('}');
    } else {
      TensorInfo t;
      t.name = key;
      std::vector<uint64_t> offs;
      while (true) {
        const std::string f = c.str();
        c.expect(':');
        if (f == "dtype") t.dtype = c.str();
        else if (f == "shape") t.shape = c.num_array();
        else if (f == "data_offsets") offs = c.num_array();
        else throw std::invalid_argument("safetensors: unknown field '" + f + "'");
        if (c.peek(',')) { ++c.p; continue; }
        break;
      }
      c.expect('}');
      if (offs.size() != 2 || offs[1] < offs[0] || 8 + n + offs[1] > mf.size())
        throw std::invalid_argument("safetensors: bad data_offsets for '" + key + "'");
      t.offset = 8 + n + offs[0];
      t.nbytes = offs[1] - offs[0];
      out.tensors.push_back(std::move(t));
    }
    if (c.peek(',')) { ++c.p; continue; }
    c.expect('}');
    break;
  }
  return out;
}

// ------------------------------------------------------------------------------ GGUF v3
static const uint32_t kGgufAlign = 32;
static uint32_t gguf_type_of(const std::string& d) {
  if (d == "F32") return 0;
  if (d == "F16") return 1;
  if (d == "BF16") return 30;
  if (d == "I8") return 24;
  if (d == "I16") return 25;
  if (d == "I32") return 26;
  if (d == "I64") return 27;
  if (d == "F64") return 28;
  throw std::invalid_argument("gguf: dtype '" + d + "' has no GGUF tensor type");
}
static std::string gguf_dtype_name(uint32_t t) {
  switch (t) {
    case 0: return "F32";
    case 1: return "F16";
    case 30: return "BF16";
    case 24: return "I8";
    case 25: return "I16";
    case 26: return "I32";
    case 27: return "I64";
    case 28: return "F64";
    default: throw std::invalid_argument("gguf: unsupported tensor type " + std::to_string(t));
  }
}
static void put_gstr(std::string& out, const std::string& s) {
  put_le<uint64_t>(out, s.size());
  out += s;
}

void gguf_write(const std::string& path, const std::vector<TensorToWrite>& tensors,
                const std::map<std::string, std::string>& metadata) {
  std::string head;
  head.append("GGUF", 4);
  put_le<uint32_t>(head, 3);
  put_le<uint64_t>(head, tensors.size());
  put_le<uint64_t>(head, metadata.size());
  for (auto& kv : metadata) {
    put_gstr(head, kv.first);
    put_le<uint32_t>(head, 8);  // GGUF_TYPE_STRING
    put_gstr(head, kv.second);
  }
  uint64_t off = 0;
  std::vector<uint64_t> offs;
  for (auto& t : tensors) {
    put_gstr(head, t.name);
    put_le<uint32_t>(head, static_cast<uint32_t>(t.shape.size()));
    for (size_t i = t.shape.size(); i-- > 0;) put_le<uint64_t>(head, t.shape[i]);  // ne[0] = innermost
    put_le<uint32_t>(head, gguf_type_of(t.dtype));
    put_le<uint64_t>(head, off);
    offs.push_back(off);
    off += (t.nbytes + kGgufAlign - 1) / kGgufAlign * kGgufAlign;
  }
  while (head.size() % kGgufAlign) head.push_back('\0');
  FILE* f = std::fopen(path.c_str(), "wb");
  if (!f) throw std::runtime_error("io failed: cannot create '" + path + "'");
  std::fwrite(head.data(), 1, head.size(), f);
  static const char zeros[kGgufAlign] = {0};
  for (auto& t : tensors) {
    if (t.nbytes) std::fwrite(t.data, 1, t.nbytes, f);
    const size_t pad = (kGgufAlign - t.nbytes % kGgufAlign) % kGgufAlign;
    if (pad) std::fwrite(zeros, 1, pad, f);
  }
  std::fclose(f);
}

TensorFile gguf_index(const std::string& path) {
  MappedFile mf(path);
  const uint8_t* b = mf.data();
  size_t cur = 0;
  auto need = [&](size_t k) {
    if (cur + k > mf.size()) throw std::invalid_argument("gguf: truncated file");
  };
  auto rd32 = [&]() { need(4); uint32_t v = get_le<uint32_t>(b + cur); cur += 4; return v; };
  auto rd64 = [&]() { need(8); uint64_t v = get_le<uint64_t>(b + cur); cur += 8; return v; };
  auto rdstr = [&]() {
    const uint64_t n = rd64();
    need(n);
    std::string s(reinterpret_cast<const char*>(b + cur), n);
    cur += n;
    return s;
  };
  need(4);
  if (std::memcmp(b, "GGUF", 4) != 0) throw std::invalid_argument("gguf: bad magic");
  cur = 4;
  const uint32_t version = rd32();
  if (version < 2 || version > 3) throw std::invalid_argument("gguf: unsupported version");
  const uint64_t n_tensors = rd64(), n_kv = rd64();
  TensorFile out;
  uint32_t align = kGgufAlign;
  static const size_t scalar_size[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
  std::function<std::string(uint32_t)> read_value = [&](uint32_t type) -> std::string {
    if (type == 8) return rdstr();
    if (type == 9) {
      const uint32_t et = rd32();
      const uint64_t n = rd64();
      std::string s = "[";
      for (uint64_t i = 0; i < n; ++i) {
        if (i) s.push_back(',');
        s += read_value(et);
      }
      return s + "]";
    }
    if (type > 12) throw std::invalid_argument("gguf: unknown value type");
    const size_t sz = scalar_size[type];
    need(sz);
    std::string s;
    switch (type) {
      case 0: s = std::to_string(b[cur]); break;
      case 1: s = std::to_string(static_cast<int8_t>(b[cur])); break;
      case 2: s = std::to_string(get_le<uint16_t>(b + cur)); break;
      case 3: s = std::to_string(static_cast<int16_t>(get_le<uint16_t>(b + cur))); break;
      case 4: s = std::to_string(get_le<uint32_t>(b + cur)); break;
      case 5: s = std::to_string(static_cast<int32_t>(get_le<uint32_t>(b + cur))); break;
      case 6: { float f; std::memcpy(&f, b + cur, 4); s = std::to_string(f); break; }
      case 7: s = b[cur] ? "true" : "false"; break;
      case 10: s = std::to_string(get_le<uint64_t>(b + cur)); break;
      case 11: s = std::to_string(static_cast<int64_t>(get_le<uint64_t>(b + cur))); break;
      case 12: { double d; std::memcpy(&d, b + cur, 8); s = std::to_string(d); break; }
    }
    cur += sz;
    return s;
  };
  for (uint64_t i = 0; i < n_kv; ++i) {
    const std::string key = rdstr();
    const uint32_t type = rd32();
    const std::string val = read_value(type);
    out.metadata[key] = val;
    if (key == "general.alignment") align = static_cast<uint32_t>(std::stoul(val));
  }
  for (uint64_t i = 0; i < n_tensors; ++i) {
    TensorInfo t;
    t.name = rdstr();
    const uint32_t nd = rd32();
    std::vector<uint64_t> ne(nd);
    for (uint32_t d = 0; d < nd; ++d) ne[d] = rd64();
    t.shape.assign(ne.rbegin(), ne.rend());
    t.dtype = gguf_dtype_name(rd32());
    t.offset = rd64();
    uint64_t numel = 1;
    for (uint64_t d : t.shape) numel *= d;
    t.nbytes = numel * dtype_size(t.dtype);
    out.tensors.push_back(std::move(t));
  }
  const uint64_t data_start = (cur + align - 1) / align * align;
  for (auto& t : out.tensors) {
    t.offset += data_start;
    if (t.offset + t.nbytes > mf.size()) throw std::invalid_argument("gguf: tensor data out of range");
  }
  return out;
}

// ------------------------------------------------------------------------------ xxHash64
static inline uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
uint64_t xxhash64(const void* data, size_t len, uint64_t seed) {
  const uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull,
                 P3 = 1609587929392839161ull, P4 = 9650029242287828579ull,
                 P5 = 2870177450012600261ull;
  const uint8_t* p = static_cast<const uint8_t*>(data);
  const uint8_t* end = p + len;
  uint64_t h;
  auto round = [&](uint64_t acc, uint64_t in) { return rotl64(acc + in * P2, 31) * P1; };
  auto merge = [&](uint64_t acc, uint64_t v) { return (acc ^ round(0, v)) * P1 + P4; };
  if (len >= 32) {
    uint64_t v1 = seed + P1 + P2, v2 = seed + P2, v3 = seed, v4 = seed - P1;
    const uint8_t* limit = end - 32;
    do {
      v1 = round(v1, get_le<uint64_t>(p)); p += 8;
      v2 = round(v2, get_le<uint64_t>(p)); p += 8;
      v3 = round(v3, get_le<uint64_t>(p)); p += 8;
      v4 = round(v4, get_le<uint64_t>(p)); p += 8;
    } while (p <= limit);
    h = rotl64(v1, 1) + rotl64(v2, 7) + rotl64(v3, 12) + rotl64(v4, 18);
    h = merge(h, v1); h = merge(h, v2); h = merge(h, v3); h = merge(h, v4);
  } else {
    h = seed + P5;
  }
  h += len;
  while (p + 8 <= end) { h ^= round(0, get_le<uint64_t>(p)); h = rotl64(h, 27) * P1 + P4; p += 8; }
  if (p + 4 <= end) { h ^= static_cast<uint64_t>(get_le<uint32_t>(p)) * P1; h = rotl64(h, 23) * P2 + P3; p += 4; }
  while (p < end) { h ^= (*p) * P5; h = rotl64(h, 11) * P1; ++p; }
  h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
  return h;
}

}  // namespace coeus
