// Checkpoint IO: the reference's `.rustllm` container (bit-exact header, little-endian fp32
// parameters, length-prefixed metadata, add-then-rotate checksum; src/core/serialization.rs),
// SafeTensors and GGUF (v3).  Readers map the file and hand out views; writers stream.
#pragma once
#include <cstdint>
#include <functional>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace coeus {

// ---------------------------------------------------------------- mmap
class MappedFile {
 public:
  explicit MappedFile(const std::string& path);
  ~MappedFile();
  MappedFile(const MappedFile&) = delete;
  const uint8_t* data() const { return data_; }
  size_t size() const { return size_; }

 private:
  int fd_ = -1;
  uint8_t* data_ = nullptr;
  size_t size_ = 0;
};

// ---------------------------------------------------------------- .rustllm
constexpr size_t kRustllmHeaderBytes = 136;

struct RustllmHeader {
  uint32_t format_version = 1;
  uint16_t ver_major = 1, ver_minor = 0, ver_patch = 0;
  uint64_t param_count = 0, param_bytes = 0, param_offset = kRustllmHeaderBytes;
  uint64_t metadata_offset = 0, metadata_size = 0, checksum = 0;
};

struct RustllmMetadata {
  std::string architecture;
  bool has_training_config = false;
  std::string training_config;
  std::vector<std::pair<std::string, std::string>> custom;
};

// c = rotl64(c + bits(p), 1) per element, in order (serialization.rs:375-385).  `seed` lets a
// stream be checksummed in pieces.
uint64_t rustllm_checksum(const float* p, size_t n, uint64_t seed = 0);
std::string rustllm_pack_header(const RustllmHeader& h);                       // 136 bytes
RustllmHeader rustllm_unpack_header(const uint8_t* bytes, size_t n);            // validates
std::string rustllm_metadata_to_bytes(const RustllmMetadata& m);
RustllmMetadata rustllm_metadata_from_bytes(const uint8_t* bytes, size_t n);

using Progress = std::function<void(size_t, size_t)>;
// Writes header | params | metadata; returns the header that was written.
RustllmHeader rustllm_write(const std::string& path, const float* params, size_t n,
                            const RustllmMetadata& meta, const Progress& progress);
// Reads and verifies; fills params.
RustllmHeader rustllm_read(const std::string& path, std::vector<float>& params,
                           RustllmMetadata& meta, const Progress& progress);

// ---------------------------------------------------------------- tensors (safetensors / gguf)
struct TensorInfo {
  std::string name;
  std::string dtype;            // "F32", "BF16", "F16", "I64", "I32", "U8"
  std::vector<uint64_t> shape;
  uint64_t offset = 0;          // byte offset of the data inside the file
  uint64_t nbytes = 0;
};

struct TensorFile {
  std::vector<TensorInfo> tensors;
  std::map<std::string, std::string> metadata;
};

struct TensorToWrite {
  std::string name;
  std::string dtype;
  std::vector<uint64_t> shape;
  const void* data;
  uint64_t nbytes;
};

size_t dtype_size(const std::string& dtype);
void safetensors_write(const std::string& path, const std::vector<TensorToWrite>& tensors,
                       const std::map<std::string, std::string>& metadata);
TensorFile safetensors_index(const std::string& path);
void gguf_write(const std::string& path, const std::vector<TensorToWrite>& tensors,
                const std::map<std::string, std::string>& metadata);
TensorFile gguf_index(const std::string& path);

uint64_t xxhash64(const void* data, size_t len, uint64_t seed = 0);

}  // namespace coeus
