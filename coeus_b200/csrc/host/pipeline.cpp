#include "pipeline.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <random>

namespace coeus {

// ------------------------------------------------------------------------------ loader
TokenBatchLoader::TokenBatchLoader(std::vector<int32_t> tokens, size_t window, size_t step,
                                   size_t batch, size_t prefetch, bool shuffle, uint64_t seed,
                                   bool drop_last)
    : tokens_(std::move(tokens)), window_(window), step_(step ? step : 1), batch_(batch),
      prefetch_(prefetch ? prefetch : 1), shuffle_(shuffle), drop_last_(drop_last), seed_(seed) {
  if (tokens_.size() >= window_)
    for (size_t s = 0; s + window_ <= tokens_.size(); s += step_) starts_.push_back(s);
  reset(0);
}

TokenBatchLoader::~TokenBatchLoader() { stop(); }

void TokenBatchLoader::stop() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    quit_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

void TokenBatchLoader::reset(uint64_t epoch) {
  stop();
  order_.resize(starts_.size());
  std::iota(order_.begin(), order_.end(), 0);
  if (shuffle_) {
    std::mt19937_64 rng(seed_ + 0x9E3779B97F4A7C15ull * (epoch + 1));
    std::shuffle(order_.begin(), order_.end(), rng);
  }
  queue_.clear();
  produce_pos_ = 0;
  consumed_ = 0;
  done_ = false;
  quit_ = false;
  thread_ = std::thread(&TokenBatchLoader::worker, this);
}

void TokenBatchLoader::seek(size_t batches_done) {
  stop();
  queue_.clear();
  produce_pos_ = std::min(order_.size(), batches_done * batch_);
  consumed_ = batches_done;
  done_ = false;
  quit_ = false;
  thread_ = std::thread(&TokenBatchLoader::worker, this);
}

void TokenBatchLoader::worker() {
  while (true) {
    size_t begin, rows;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [&] { return quit_ || queue_.size() < prefetch_; });
      if (quit_) return;
      begin = produce_pos_;
      rows = std::min(batch_, order_.size() - begin);
      if (rows == 0 || (drop_last_ && rows < batch_)) {
        done_ = true;
        cv_.notify_all();
        return;
      }
      produce_pos_ += rows;
    }
    std::vector<int64_t> buf(rows * window_);
    for (size_t r = 0; r < rows; ++r) {
      const int32_t* src = tokens_.data() + starts_[order_[begin + r]];
      for (size_t j = 0; j < window_; ++j) buf[r * window_ + j] = src[j];
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      queue_.push_back(std::move(buf));
    }
    cv_.notify_all();
  }
}

size_t TokenBatchLoader::next(int64_t* out) {
  std::vector<int64_t> buf;
  {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !queue_.empty() || done_; });
    if (queue_.empty()) return 0;
    buf = std::move(queue_.front());
    queue_.pop_front();
    ++consumed_;
  }
  cv_.notify_all();
  std::memcpy(out, buf.data(), buf.size() * sizeof(int64_t));
  return buf.size() / window_;
}

// ------------------------------------------------------------------------------ suffix array
// Prefix doubling with a radix-free comparison sort per round: O(n log^2 n), the algorithm the
// reference implements (under a comment that calls it DC3; src/foundation/iterator.rs:1019-1058).
std::vector<int64_t> suffix_array(const std::string& text) {
  const size_t n = text.size();
  std::vector<int64_t> sa(n), rank(n), tmp(n);
  for (size_t i = 0; i < n; ++i) { sa[i] = static_cast<int64_t>(i); rank[i] = static_cast<unsigned char>(text[i]); }
  for (size_t k = 1; n > 1; k <<= 1) {
    auto key = [&](int64_t i) {
      return std::make_pair(rank[i], static_cast<size_t>(i) + k < n ? rank[i + k] : int64_t(-1));
    };
    std::sort(sa.begin(), sa.end(), [&](int64_t a, int64_t b) { return key(a) < key(b); });
    tmp[sa[0]] = 0;
    for (size_t j = 1; j < n; ++j) tmp[sa[j]] = tmp[sa[j - 1]] + (key(sa[j - 1]) < key(sa[j]) ? 1 : 0);
    rank = tmp;
    if (rank[sa[n - 1]] == static_cast<int64_t>(n) - 1) break;
  }
  return sa;
}

// ------------------------------------------------------------------------------ bloom
NativeBloom::NativeBloom(size_t expected, double fp_rate) {
  const double bits_per_item = -(std::log(fp_rate) / (std::log(2.0) * std::log(2.0)));
  nbits_ = static_cast<size_t>(std::ceil(static_cast<double>(expected) * bits_per_item));
  if (nbits_ == 0) nbits_ = 1;
  k_ = static_cast<size_t>(std::ceil(bits_per_item * std::log(2.0)));
  bits_.assign((nbits_ + 63) / 64, 0);
}
static size_t murmur_like(const std::string& data, size_t seed) {
  size_t h = seed;
  for (unsigned char b : data) {
    h ^= b;
    h *= 0x5bd1e995ull;
    h ^= h >> 15;
  }
  return h;
}
size_t NativeBloom::hash(const std::string& item, size_t k) const {
  const size_t h1 = murmur_like(item, 0), h2 = murmur_like(item, h1);
  return (h1 + k * h2) % nbits_;
}
void NativeBloom::insert(const std::string& item) {
  for (size_t k = 0; k < k_; ++k) {
    const size_t b = hash(item, k);
    bits_[b >> 6] |= 1ull << (b & 63);
  }
}
bool NativeBloom::contains(const std::string& item) const {
  for (size_t k = 0; k < k_; ++k) {
    const size_t b = hash(item, k);
    if (!(bits_[b >> 6] >> (b & 63) & 1ull)) return false;
  }
  return true;
}
size_t NativeBloom::popcount() const {
  size_t n = 0;
  for (uint64_t w : bits_) n += static_cast<size_t>(__builtin_popcountll(w));
  return n;
}

// ------------------------------------------------------------------------------ arena
NativeArena::NativeArena(size_t chunk_size, size_t alignment)
    : chunk_size_(chunk_size), alignment_(alignment) {}
NativeArena::~NativeArena() {
  for (auto& c : chunks_) std::free(c.data);
}
void* NativeArena::alloc(size_t bytes) {
  while (true) {
    if (current_ < chunks_.size()) {
      Chunk& c = chunks_[current_];
      const size_t start = (c.used + alignment_ - 1) / alignment_ * alignment_;
      if (start + bytes <= c.size) {
        c.used = start + bytes;
        stats_.allocated_bytes += bytes;
        stats_.used_bytes += bytes;
        stats_.allocation_count += 1;
        stats_.peak_bytes = std::max(stats_.peak_bytes, stats_.used_bytes);
        return c.data + start;
      }
      ++current_;
      continue;
    }
    const size_t size = std::max(chunk_size_, bytes + alignment_);
    void* p = nullptr;
    if (posix_memalign(&p, std::max<size_t>(alignment_, sizeof(void*)), size) != 0) return nullptr;
    chunks_.push_back({static_cast<uint8_t*>(p), size, 0});
    current_ = chunks_.size() - 1;
  }
}
void NativeArena::reset() {
  for (auto& c : chunks_) c.used = 0;
  current_ = 0;
  stats_.deallocated_bytes += stats_.used_bytes;
  stats_.deallocation_count += 1;
  stats_.used_bytes = 0;
}
size_t NativeArena::capacity() const {
  size_t n = 0;
  for (auto& c : chunks_) n += c.size;
  return n;
}
size_t NativeArena::used() const {
  size_t n = 0;
  for (auto& c : chunks_) n += c.used;
  return n;
}

}  // namespace coeus
