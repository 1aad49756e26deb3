// Native pieces of the data path and the utility algorithms: token-stream windows / chunks /
// batches with a background prefetch thread (the device-side use of the reference's iterator
// adapters, src/foundation/iterator.rs), suffix array, Bloom filter, arena and pool with
// statistics (src/foundation/memory.rs).
#pragma once
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace coeus {

// ---- token windows: rows of `window` ids taken every `step` ids from one long stream, grouped
// into batches of `batch` rows, produced ahead of the consumer by a worker thread.
class TokenBatchLoader {
 public:
  TokenBatchLoader(std::vector<int32_t> tokens, size_t window, size_t step, size_t batch,
                   size_t prefetch, bool shuffle, uint64_t seed, bool drop_last);
  ~TokenBatchLoader();
  // Copies the next batch (rows * window ids, int64 for the embedding kernel) into out; returns
  // the number of rows, 0 at the end of the epoch.
  size_t next(int64_t* out);
  void reset(uint64_t epoch);
  size_t num_windows() const { return starts_.size(); }
  size_t cursor() const { return consumed_; }
  void seek(size_t batches_done);

 private:
  void worker();
  void stop();
  std::vector<int32_t> tokens_;
  std::vector<size_t> starts_, order_;
  size_t window_, step_, batch_, prefetch_;
  bool shuffle_, drop_last_;
  uint64_t seed_;
  size_t produce_pos_ = 0, consumed_ = 0;
  std::deque<std::vector<int64_t>> queue_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::thread thread_;
  bool done_ = false, quit_ = false;
};

std::vector<int64_t> suffix_array(const std::string& text);

class NativeBloom {
 public:
  NativeBloom(size_t expected, double fp_rate);
  void insert(const std::string& item);
  bool contains(const std::string& item) const;
  size_t bit_count() const { return nbits_; }
  size_t popcount() const;
  size_t hash_count() const { return k_; }

 private:
  size_t hash(const std::string& item, size_t k) const;
  std::vector<uint64_t> bits_;
  size_t nbits_, k_;
};

struct NativeMemoryStats {
  size_t allocated_bytes = 0, deallocated_bytes = 0, used_bytes = 0, peak_bytes = 0,
         allocation_count = 0, deallocation_count = 0;
};

// Chunked bump allocator over host memory (optionally page-locked by the caller).
class NativeArena {
 public:
  explicit NativeArena(size_t chunk_size, size_t alignment = 64);
  ~NativeArena();
  void* alloc(size_t bytes);
  void reset();
  size_t capacity() const;
  size_t used() const;
  const NativeMemoryStats& stats() const { return stats_; }

 private:
  struct Chunk { uint8_t* data; size_t size, used; };
  std::vector<Chunk> chunks_;
  size_t chunk_size_, alignment_, current_ = 0;
  NativeMemoryStats stats_;
};

}  // namespace coeus
