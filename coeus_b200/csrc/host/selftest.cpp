// Native self-test of the host library, meant to be built with sanitizers
// (-fsanitize=address,undefined or -fsanitize=thread): it drives the tokenizers, the file
// formats (including damaged inputs), the CPU oracle and the threaded batch loader without any
// Python in the process, so that a report points at this code only.  Exits 0 when every check
// holds, prints the failed check and exits 1 otherwise.
//
// The reference relies on the Rust type system for memory and thread safety of the same
// components (src/foundation/memory.rs:223-228 asserts Send/Sync by hand; PRD.md:220 lists
// sanitizers as a mitigation without configuring any).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "io.hpp"
#include "oracle.hpp"
#include "pipeline.hpp"
#include "tokenizers.hpp"

using namespace coeus;

static int g_failed = 0;
#define CHECK(cond)                                                      \
  do {                                                                   \
    if (!(cond)) {                                                       \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++g_failed;                                                        \
    }                                                                    \
  } while (0)

template <class F>
static bool throws(F&& f) {
  try {
    f();
  } catch (const std::exception&) {
    return true;
  }
  return false;
}

static void test_tokenizers() {
  BpeTokenizer bpe;
  std::vector<std::string> corpus = {"the cat sat on the mat", "the dog sat on the log",
                                     "na\xc3\xafve caf\xc3\xa9 \xe6\x97\xa5\xe6\x9c\xac"};
  bpe.train(corpus, 40);
  CHECK(bpe.num_merges() > 0);
  static const char malformed[] = "bad \xff\xfe bytes \xc3";   // ends inside a 2-byte sequence
  const std::string texts[] = {"the cat sat", "", "   ", "unseen w\xc3\xb6rds \xf0\x9f\x98\x80",
                               std::string(malformed, sizeof(malformed) - 1)};
  for (const std::string& t : texts) {
    std::vector<uint32_t> ids;
    std::vector<std::string> strs;
    bpe.encode(t, ids, &strs);
    CHECK(ids.size() == strs.size());
    (void)bpe.decode_ids(ids);
    (void)bpe.decode_strings(strs);
  }
  std::vector<uint32_t> ids;
  bpe.encode("the cat sat on the mat", ids);
  CHECK(bpe.decode_ids(ids) == "the cat sat on the mat");
  const uint32_t id = bpe.add_token("<extra>");
  std::string back;
  CHECK(bpe.token_from_id(id, back) && back == "<extra>");
  CHECK(bpe.remove_token("<extra>") && !bpe.contains_token("<extra>"));
  CHECK(!bpe.token_from_id(0xFFFFFFF0u, back));
  if (bpe.num_merges() > 0) (void)bpe.merge_at(bpe.num_merges() - 1);
  bpe.clear_cache();
  {
    // replaying the merges on a fresh tokenizer reproduces the ids
    std::vector<std::pair<std::string, std::string>> pairs;
    for (size_t i = 0; i < bpe.num_merges(); ++i) pairs.push_back(bpe.merge_at(i));
    BpeTokenizer again;
    again.load_merges(pairs);
    std::vector<uint32_t> x, y;
    bpe.encode("the cat sat on the caf\xc3\xa9", x);
    again.encode("the cat sat on the caf\xc3\xa9", y);
    CHECK(x == y && again.vocab_size() == bpe.vocab_size());
  }

  WordPieceTokenizer wp;
  uint32_t next = 100;
  for (const char* t : {"un", "##aff", "##able", "the", "##s", "caf", "##e\xcc\x81"})
    wp.add_token(t, next++);
  auto e = wp.encode("unaffable the thes caf\xc3\xa9 zzz");
  CHECK(e.size() >= 2);
  (void)wp.tokenize_word("unaffable");
  (void)wp.tokenize_word("");
  uint32_t mid;
  size_t chars;
  (void)wp.longest_match("unaffable", mid, chars);
  CHECK(is_nfd(nfd("caf\xc3\xa9 \xc7\x96")));
  CHECK(unicode_words("can't stop, 3.14 ok").size() >= 3);
  BasicTokenizer basic;
  CHECK(basic.tokenize(" a\tb\xe2\x80\x83" "c ").size() == 3);
}

static void test_formats(const std::string& dir) {
  std::vector<float> p(1000);
  for (size_t i = 0; i < p.size(); ++i) p[i] = std::sin(0.1f * static_cast<float>(i));
  RustllmMetadata meta;
  meta.architecture = "transformer";
  meta.has_training_config = true;
  meta.training_config = "{\"lr\": 0.1}";
  meta.custom = {{"k", "v"}, {"", ""}};
  const std::string path = dir + "/m.rustllm";
  size_t calls = 0;
  rustllm_write(path, p.data(), p.size(), meta, [&](size_t, size_t) { ++calls; });
  std::vector<float> q;
  RustllmMetadata m2;
  const RustllmHeader h = rustllm_read(path, q, m2, nullptr);
  CHECK(h.param_count == p.size() && q == p && m2.architecture == "transformer");
  CHECK(m2.custom.size() == 2 && m2.training_config == meta.training_config);
  CHECK(rustllm_checksum(p.data(), p.size()) == h.checksum);
  // damaged files: flipped payload byte, truncated file, truncated header, truncated metadata
  {
    std::string bytes;
    {
      std::ifstream f(path, std::ios::binary);
      bytes.assign(std::istreambuf_iterator<char>(f), {});
    }
    std::string bad = bytes;
    bad[kRustllmHeaderBytes + 17] ^= 0x40;
    std::ofstream(dir + "/flip.rustllm", std::ios::binary) << bad;
    CHECK(throws([&] { rustllm_read(dir + "/flip.rustllm", q, m2, nullptr); }));
    std::ofstream(dir + "/cut.rustllm", std::ios::binary) << bytes.substr(0, bytes.size() / 2);
    CHECK(throws([&] { rustllm_read(dir + "/cut.rustllm", q, m2, nullptr); }));
    CHECK(throws([&] {
      rustllm_unpack_header(reinterpret_cast<const uint8_t*>(bytes.data()), 20);
    }));
    const std::string mb = rustllm_metadata_to_bytes(meta);
    for (size_t cut = 0; cut < mb.size(); cut += 3)
      (void)throws([&] {
        rustllm_metadata_from_bytes(reinterpret_cast<const uint8_t*>(mb.data()), cut);
      });
  }
  std::vector<uint16_t> half(64, 0x3f80);
  std::vector<TensorToWrite> ts = {
      {"a.weight", "F32", {10, 100}, p.data(), p.size() * 4},
      {"b", "BF16", {64}, half.data(), half.size() * 2},
  };
  safetensors_write(dir + "/t.safetensors", ts, {{"format", "pt"}});
  const TensorFile sf = safetensors_index(dir + "/t.safetensors");
  CHECK(sf.tensors.size() == 2);
  gguf_write(dir + "/t.gguf", ts, {{"general.architecture", "llama"}});
  const TensorFile gf = gguf_index(dir + "/t.gguf");
  CHECK(gf.tensors.size() == 2);
  {
    MappedFile mf(dir + "/t.safetensors");
    (void)mf;
  }
  std::ofstream(dir + "/junk.safetensors", std::ios::binary) << std::string(5, 'x');
  CHECK(throws([&] { safetensors_index(dir + "/junk.safetensors"); }));
  std::ofstream(dir + "/junk.gguf", std::ios::binary) << std::string("GGUF\x03\x00\x00", 7);
  CHECK(throws([&] { gguf_index(dir + "/junk.gguf"); }));
  CHECK(throws([&] { MappedFile missing(dir + "/does-not-exist"); }));
  CHECK(xxhash64("abc", 3) != xxhash64("abd", 3));
  CHECK(dtype_size("BF16") == 2);
}

static void test_oracle() {
  OracleConfig c{32, 2, 2, 64, 50, 16, 1e-5f, true};
  const size_t n = oracle_param_count(c);
  std::vector<float> p(n);
  oracle_sin_init(p.data(), n, c.hidden);
  const int64_t ids[5] = {1, 7, 49, 0, 3};
  for (bool compat : {false, true}) {
    const std::vector<float> last = oracle_forward(p.data(), n, c, ids, 5, compat, false);
    const std::vector<float> all = oracle_forward(p.data(), n, c, ids, 5, compat, true);
    CHECK(last.size() == c.vocab && all.size() == 5 * c.vocab);
    for (size_t v = 0; v < c.vocab; ++v) CHECK(std::fabs(last[v] - all[4 * c.vocab + v]) < 1e-5f);
  }
  const int64_t bad[2] = {1, 50};
  CHECK(throws([&] { oracle_forward(p.data(), n, c, bad, 2, false, false); }));
}

static void test_pipeline() {
  std::vector<int32_t> toks(1003);
  for (size_t i = 0; i < toks.size(); ++i) toks[i] = static_cast<int32_t>(i);
  for (bool shuffle : {false, true}) {
    TokenBatchLoader ld(toks, 17, 16, 4, 3, shuffle, 7, false);
    std::vector<int64_t> out(4 * 17);
    for (uint64_t epoch = 0; epoch < 3; ++epoch) {
      ld.reset(epoch);
      size_t rows = 0, got;
      while ((got = ld.next(out.data())) != 0) {
        rows += got;
        for (size_t r = 0; r < got; ++r)
          for (size_t j = 1; j < 17; ++j) CHECK(out[r * 17 + j] == out[r * 17] + (int64_t)j);
      }
      CHECK(rows == ld.num_windows());
    }
    ld.reset(1);
    ld.seek(2);
    CHECK(ld.next(out.data()) > 0);
    // destroyed while its worker may still be producing
  }
  {
    // several loaders driven from several threads at once
    std::vector<std::thread> th;
    for (int t = 0; t < 4; ++t)
      th.emplace_back([&toks, t] {
        TokenBatchLoader ld(toks, 9, 8, 8, 2, true, 100 + t, true);
        std::vector<int64_t> out(8 * 9);
        size_t n = 0;
        while (ld.next(out.data()) != 0) ++n;
        if (n == 0) std::abort();
      });
    for (auto& x : th) x.join();
  }
  const std::string text = "banana bandana";
  const std::vector<int64_t> sa = suffix_array(text);
  CHECK(sa.size() == text.size());
  for (size_t i = 1; i < sa.size(); ++i) CHECK(text.substr(sa[i - 1]) < text.substr(sa[i]));
  CHECK(suffix_array("").empty());
  NativeBloom bloom(100, 0.01);
  for (int i = 0; i < 100; ++i) bloom.insert("item" + std::to_string(i));
  for (int i = 0; i < 100; ++i) CHECK(bloom.contains("item" + std::to_string(i)));
  CHECK(bloom.popcount() > 0 && bloom.popcount() <= bloom.bit_count());
  NativeArena arena(4096, 64);
  for (size_t sz : {1u, 63u, 64u, 4000u, 9000u, 0u}) {
    void* ptr = arena.alloc(sz);
    CHECK(ptr != nullptr && reinterpret_cast<uintptr_t>(ptr) % 64 == 0);
    if (sz) std::memset(ptr, 0xab, sz);
  }
  CHECK(arena.used() <= arena.capacity() && arena.stats().allocation_count == 6);
  arena.reset();
  CHECK(arena.used() == 0);
}

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  try {
    test_tokenizers();
    test_formats(dir);
    test_oracle();
    test_pipeline();
  } catch (const std::exception& e) {
    std::fprintf(stderr, "unexpected exception: %s\n", e.what());
    return 1;
  }
  if (g_failed) return 1;
  std::puts("host selftest ok");
  return 0;
}
