// pybind11 module `_coeus_host`: tokenizers, checkpoint IO, data pipeline, text algorithms, arena
// and the CPU oracle.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <thread>

#include "io.hpp"
#include "oracle.hpp"
#include "pipeline.hpp"
#include "tokenizers.hpp"

namespace py = pybind11;
using namespace coeus;

static py::dict tensor_file_to_py(const TensorFile& tf) {
  py::list ts;
  for (auto& t : tf.tensors) {
    py::dict d;
    d["name"] = t.name;
    d["dtype"] = t.dtype;
    d["shape"] = t.shape;
    d["offset"] = t.offset;
    d["nbytes"] = t.nbytes;
    ts.append(d);
  }
  py::dict out;
  out["tensors"] = ts;
  out["metadata"] = tf.metadata;
  return out;
}

static std::vector<TensorToWrite> tensors_from_py(const py::list& items, std::vector<py::buffer_info>& keep) {
  std::vector<TensorToWrite> out;
  for (auto item : items) {
    auto tup = item.cast<py::tuple>();  // (name, dtype, shape, buffer)
    py::buffer buf = tup[3].cast<py::buffer>();
    keep.push_back(buf.request());
    TensorToWrite t;
    t.name = tup[0].cast<std::string>();
    t.dtype = tup[1].cast<std::string>();
    t.shape = tup[2].cast<std::vector<uint64_t>>();
    t.data = keep.back().ptr;
    t.nbytes = static_cast<uint64_t>(keep.back().size * keep.back().itemsize);
    out.push_back(t);
  }
  return out;
}

PYBIND11_MODULE(_coeus_host, m) {
  m.doc() = "native host components of coeus_b200";

  // ------------------------------------------------------------------ tokenizers
  m.def("split_whitespace", [](const std::string& s) {
    std::vector<std::string> out;
    for (auto v : split_whitespace(s)) out.emplace_back(v);
    return out;
  });
  m.def("nfd", [](const std::string& s) { return nfd(s); });
  m.def("is_nfd", [](const std::string& s) { return is_nfd(s); });
  m.def("unicode_words", [](const std::string& s) { return unicode_words(s); });

  py::class_<BpeTokenizer>(m, "BpeTokenizer")
      .def(py::init<>())
      .def("train", &BpeTokenizer::train, py::call_guard<py::gil_scoped_release>())
      .def("load_merges", &BpeTokenizer::load_merges)
      .def("encode", [](BpeTokenizer& t, const std::string& text) {
        std::vector<uint32_t> ids;
        { py::gil_scoped_release r; t.encode(text, ids); }
        return py::array_t<uint32_t>(static_cast<py::ssize_t>(ids.size()), ids.data());
      })
      .def("encode_with_strings", [](BpeTokenizer& t, const std::string& text) {
        std::vector<uint32_t> ids;
        std::vector<std::string> strs;
        t.encode(text, ids, &strs);
        py::list ps;  // token strings may hold lone control bytes only (always valid UTF-8)
        for (auto& s : strs) ps.append(py::str(s));
        return py::make_tuple(ids, ps);
      })
      .def("encode_batch", [](BpeTokenizer& t, const std::vector<std::string>& texts) {
        std::vector<std::vector<uint32_t>> rows(texts.size());
        { py::gil_scoped_release r; for (size_t i = 0; i < texts.size(); ++i) t.encode(texts[i], rows[i]); }
        return rows;
      })
      .def("decode_strings", &BpeTokenizer::decode_strings)
      .def("decode_ids", &BpeTokenizer::decode_ids, py::call_guard<py::gil_scoped_release>())
      .def("decode_ids_bytes", [](const BpeTokenizer& t, const std::vector<uint32_t>& ids) {
        return py::bytes(t.decode_ids_bytes(ids));
      })
      .def("vocab_size", &BpeTokenizer::vocab_size)
      .def("add_token", &BpeTokenizer::add_token)
      .def("remove_token", &BpeTokenizer::remove_token)
      .def("contains_token", &BpeTokenizer::contains_token)
      .def("token_from_id", [](const BpeTokenizer& t, uint32_t id) -> py::object {
        std::string s;
        if (!t.token_from_id(id, s)) return py::none();
        return py::str(s);
      })
      .def("id_from_token", [](const BpeTokenizer& t, const std::string& tok) -> py::object {
        uint32_t id;
        if (!t.id_from_token(tok, id)) return py::none();
        return py::int_(id);
      })
      .def("num_merges", &BpeTokenizer::num_merges)
      .def("merge_at", &BpeTokenizer::merge_at)
      .def("merge_at_bytes", [](const BpeTokenizer& t, size_t i) {
        auto pr = t.merge_at(i);
        return py::make_tuple(py::bytes(pr.first), py::bytes(pr.second));
      });

  py::class_<WordPieceTokenizer>(m, "WordPieceTokenizer")
      .def(py::init<>())
      .def("add_token", &WordPieceTokenizer::add_token)
      .def("encode", &WordPieceTokenizer::encode)
      .def("tokenize_word", [](const WordPieceTokenizer& t, const std::string& w) { return t.tokenize_word(w); })
      .def("decode_strings", &WordPieceTokenizer::decode_strings)
      .def("vocab_size", &WordPieceTokenizer::vocab_size)
      .def("id_to_token", [](const WordPieceTokenizer& t, uint32_t id) -> py::object {
        std::string s;
        if (!t.id_to_token(id, s)) return py::none();
        return py::str(s);
      })
      .def("token_to_id", [](const WordPieceTokenizer& t, const std::string& s) -> py::object {
        uint32_t id;
        if (!t.token_to_id(s, id)) return py::none();
        return py::int_(id);
      })
      .def("longest_match", [](const WordPieceTokenizer& t, const std::string& s) -> py::object {
        uint32_t id;
        size_t chars;
        if (!t.longest_match(s, id, chars)) return py::none();
        return py::make_tuple(id, chars);
      });

  // ------------------------------------------------------------------ .rustllm
  m.def("rustllm_checksum", [](py::array_t<float, py::array::c_style | py::array::forcecast> a, uint64_t seed) {
    py::gil_scoped_release r;
    return rustllm_checksum(a.data(), static_cast<size_t>(a.size()), seed);
  }, py::arg("params"), py::arg("seed") = 0);
  m.def("rustllm_pack_header", [](uint64_t param_count, uint64_t metadata_offset, uint64_t metadata_size,
                                  uint64_t checksum, std::tuple<int, int, int> ver) {
    RustllmHeader h;
    h.param_count = param_count;
    h.param_bytes = 4 * param_count;
    h.metadata_offset = metadata_offset;
    h.metadata_size = metadata_size;
    h.checksum = checksum;
    h.ver_major = static_cast<uint16_t>(std::get<0>(ver));
    h.ver_minor = static_cast<uint16_t>(std::get<1>(ver));
    h.ver_patch = static_cast<uint16_t>(std::get<2>(ver));
    return py::bytes(rustllm_pack_header(h));
  });
  auto header_to_py = [](const RustllmHeader& h) {
    py::dict d;
    d["format_version"] = h.format_version;
    d["model_version"] = py::make_tuple(h.ver_major, h.ver_minor, h.ver_patch);
    d["param_count"] = h.param_count;
    d["param_bytes"] = h.param_bytes;
    d["param_offset"] = h.param_offset;
    d["metadata_offset"] = h.metadata_offset;
    d["metadata_size"] = h.metadata_size;
    d["checksum"] = h.checksum;
    return d;
  };
  m.def("rustllm_unpack_header", [header_to_py](py::bytes b) {
    const std::string s = b;
    return header_to_py(rustllm_unpack_header(reinterpret_cast<const uint8_t*>(s.data()), s.size()));
  });
  auto meta_from_py = [](const std::string& arch, py::object training, const std::vector<std::pair<std::string, std::string>>& custom) {
    RustllmMetadata mm;
    mm.architecture = arch;
    mm.has_training_config = !training.is_none();
    if (mm.has_training_config) mm.training_config = training.cast<std::string>();
    mm.custom = custom;
    return mm;
  };
  auto meta_to_py = [](const RustllmMetadata& mm) {
    py::object tc = py::none();
    if (mm.has_training_config) tc = py::str(mm.training_config);
    return py::make_tuple(mm.architecture, tc, mm.custom);
  };
  m.def("rustllm_metadata_to_bytes", [meta_from_py](const std::string& arch, py::object training,
                                                    const std::vector<std::pair<std::string, std::string>>& custom) {
    return py::bytes(rustllm_metadata_to_bytes(meta_from_py(arch, training, custom)));
  });
  m.def("rustllm_metadata_from_bytes", [meta_to_py](py::bytes b) {
    const std::string s = b;
    return meta_to_py(rustllm_metadata_from_bytes(reinterpret_cast<const uint8_t*>(s.data()), s.size()));
  });
  m.def("rustllm_write", [meta_from_py, header_to_py](const std::string& path,
                                                      py::array_t<float, py::array::c_style | py::array::forcecast> params,
                                                      const std::string& arch, py::object training,
                                                      const std::vector<std::pair<std::string, std::string>>& custom,
                                                      py::object progress) {
    Progress cb;
    if (!progress.is_none()) cb = [progress](size_t a, size_t b) { progress(a, b); };
    return header_to_py(rustllm_write(path, params.data(), static_cast<size_t>(params.size()),
                                      meta_from_py(arch, training, custom), cb));
  });
  m.def("rustllm_read", [meta_to_py, header_to_py](const std::string& path, py::object progress) {
    Progress cb;
    if (!progress.is_none()) cb = [progress](size_t a, size_t b) { progress(a, b); };
    std::vector<float> params;
    RustllmMetadata mm;
    RustllmHeader h = rustllm_read(path, params, mm, cb);
    py::array_t<float> arr(static_cast<py::ssize_t>(params.size()));
    std::memcpy(arr.mutable_data(), params.data(), params.size() * 4);
    return py::make_tuple(header_to_py(h), arr, meta_to_py(mm));
  });

  // ------------------------------------------------------------------ safetensors / gguf
  m.def("safetensors_write", [](const std::string& path, py::list items, const std::map<std::string, std::string>& meta) {
    std::vector<py::buffer_info> keep;
    keep.reserve(items.size());
    auto ts = tensors_from_py(items, keep);
    safetensors_write(path, ts, meta);
  });
  m.def("safetensors_index", [](const std::string& path) { return tensor_file_to_py(safetensors_index(path)); });
  m.def("gguf_write", [](const std::string& path, py::list items, const std::map<std::string, std::string>& meta) {
    std::vector<py::buffer_info> keep;
    keep.reserve(items.size());
    auto ts = tensors_from_py(items, keep);
    gguf_write(path, ts, meta);
  });
  m.def("gguf_index", [](const std::string& path) { return tensor_file_to_py(gguf_index(path)); });
  m.def("xxhash64", [](py::buffer b, uint64_t seed) {
    py::buffer_info info = b.request();
    return xxhash64(info.ptr, static_cast<size_t>(info.size * info.itemsize), seed);
  }, py::arg("data"), py::arg("seed") = 0);

  // ------------------------------------------------------------------ data pipeline / algorithms
  py::class_<TokenBatchLoader>(m, "TokenBatchLoader")
      .def(py::init([](py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens, size_t window,
                       size_t step, size_t batch, size_t prefetch, bool shuffle, uint64_t seed, bool drop_last) {
        std::vector<int32_t> v(tokens.data(), tokens.data() + tokens.size());
        return new TokenBatchLoader(std::move(v), window, step, batch, prefetch, shuffle, seed, drop_last);
      }), py::arg("tokens"), py::arg("window"), py::arg("step"), py::arg("batch"), py::arg("prefetch") = 2,
           py::arg("shuffle") = false, py::arg("seed") = 0, py::arg("drop_last") = true)
      .def("next_into", [](TokenBatchLoader& l, py::array_t<int64_t, py::array::c_style> out) {
        int64_t* p = out.mutable_data();
        py::gil_scoped_release r;
        return l.next(p);
      })
      .def("reset", &TokenBatchLoader::reset)
      .def("seek", &TokenBatchLoader::seek)
      .def("num_windows", &TokenBatchLoader::num_windows)
      .def("cursor", &TokenBatchLoader::cursor);

  m.def("suffix_array", [](const std::string& s) { return suffix_array(s); });
  py::class_<NativeBloom>(m, "Bloom")
      .def(py::init<size_t, double>())
      .def("insert", &NativeBloom::insert)
      .def("contains", &NativeBloom::contains)
      .def("bit_count", &NativeBloom::bit_count)
      .def("popcount", &NativeBloom::popcount)
      .def("hash_count", &NativeBloom::hash_count);
  py::class_<NativeArena>(m, "Arena")
      .def(py::init<size_t, size_t>(), py::arg("chunk_size"), py::arg("alignment") = 64)
      .def("alloc", [](NativeArena& a, size_t bytes) {
        void* p = a.alloc(bytes);
        if (!p) throw std::bad_alloc();
        return py::memoryview::from_memory(p, static_cast<py::ssize_t>(bytes));
      }, py::keep_alive<0, 1>())
      .def("reset", &NativeArena::reset)
      .def("capacity", &NativeArena::capacity)
      .def("used", &NativeArena::used)
      .def("stats", [](const NativeArena& a) {
        const auto& s = a.stats();
        py::dict d;
        d["allocated_bytes"] = s.allocated_bytes;
        d["deallocated_bytes"] = s.deallocated_bytes;
        d["used_bytes"] = s.used_bytes;
        d["peak_bytes"] = s.peak_bytes;
        d["allocation_count"] = s.allocation_count;
        d["deallocation_count"] = s.deallocation_count;
        return d;
      });

  // ------------------------------------------------------------------ oracle
  m.def("oracle_param_count", [](size_t hidden, size_t layers, size_t heads, size_t inter, size_t vocab,
                                 size_t max_seq, bool use_bias) {
    return oracle_param_count(OracleConfig{hidden, layers, heads, inter, vocab, max_seq, 1e-5f, use_bias});
  });
  m.def("oracle_sin_init", [](size_t n, size_t hidden) {
    py::array_t<float> out(static_cast<py::ssize_t>(n));
    float* p = out.mutable_data();
    { py::gil_scoped_release r; oracle_sin_init(p, n, hidden); }
    return out;
  });
  m.def("oracle_forward", [](py::array_t<float, py::array::c_style | py::array::forcecast> params, size_t hidden,
                             size_t layers, size_t heads, size_t inter, size_t vocab, size_t max_seq, float eps,
                             bool use_bias, py::array_t<int64_t, py::array::c_style | py::array::forcecast> ids,
                             bool ref_compat, bool all_positions) {
    OracleConfig c{hidden, layers, heads, inter, vocab, max_seq, eps, use_bias};
    std::vector<float> out;
    const float* pp = params.data();
    const size_t np = static_cast<size_t>(params.size());
    const int64_t* ip = ids.data();
    const size_t S = static_cast<size_t>(ids.size());
    { py::gil_scoped_release r; out = oracle_forward(pp, np, c, ip, S, ref_compat, all_positions); }
    py::array_t<float> arr(static_cast<py::ssize_t>(out.size()));
    std::memcpy(arr.mutable_data(), out.data(), out.size() * 4);
    return arr;
  }, py::arg("params"), py::arg("hidden"), py::arg("layers"), py::arg("heads"), py::arg("intermediate"),
     py::arg("vocab"), py::arg("max_seq"), py::arg("eps"), py::arg("use_bias"), py::arg("ids"),
     py::arg("ref_compat") = false, py::arg("all_positions") = false);
}
