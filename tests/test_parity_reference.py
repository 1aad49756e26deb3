"""The reference's own unit and integration assertions, restated against this package's API
(same inputs, same expected values).  Source of each group is named in its docstring."""
import io
import threading

import numpy as np
import pytest

from coeus_b200.prelude import *  # noqa: F401,F403
from coeus_b200.core.config import ConfigBuilder, ConfigStore, ConfigValue, PluginConfigManager
from coeus_b200.core.plugin import PluginCapabilities, PluginEntry, PluginState
from coeus_b200.core.serialization import (ModelHeader, ModelMetadata, ParameterSerializer,
                                           calculate_checksum)
from coeus_b200.core.tokenizer import (PaddingStrategy, PositionedToken, StringToken,
                                       TokenizerConfig, TruncationStrategy)
from coeus_b200.core.traits import Identity, Process
from coeus_b200.foundation import iterator as it
from coeus_b200.foundation.error import (CompositeError, ErrorContext, ProcessingError,
                                         error_context, internal_error, invalid_input,
                                         limit_exceeded)
from coeus_b200.foundation.memory import (Arena, BumpAllocator, CowStr, Pool, StringInterner,
                                          TrackingArena, ZeroCopyStringBuilder)
from coeus_b200.foundation.types import Shape, Version
from coeus_b200.models.config import BasicModelConfig, Transformer250MConfig
from coeus_b200.plugins.builtin import (BasicLoaderPlugin, BasicModelPlugin, BasicTokenizer,
                                        BasicTokenizerPlugin, BpeTokenizer, BpeTokenizerPlugin,
                                        TransformerModelPlugin, WordPieceTokenizer,
                                        WordPieceTokenizerPlugin)


# ------------------------------------------------------------------ src/foundation/iterator.rs
def test_windows_chunks_stride():
    assert it.Iter([1, 2, 3, 4, 5]).windows(3).collect() == [(1, 2, 3), (2, 3, 4), (3, 4, 5)]
    assert it.Iter([1, 2, 3, 4, 5, 6]).windows_step(3, 2).collect()[:2] == [(1, 2, 3), (3, 4, 5)]
    assert it.Iter([1, 2, 3, 4, 5, 6, 7]).chunks(3).collect() == [[1, 2, 3], [4, 5, 6], [7]]
    assert it.Iter([1, 2, 3, 4, 5, 6]).stride(2).collect() == [1, 3, 5]


def test_zero_copy_tokenizer_and_split():
    assert list(it.ZeroCopyTokenizer("hello world rust", " ")) == ["hello", "world", "rust"]
    assert list(it.ZeroCopySplit("hello,world,rust", ",")) == ["hello", "world", "rust"]


def test_slice_windows():
    data = [1, 2, 3, 4, 5, 6, 7, 8]
    w = list(it.slice_windows(data, 3))
    assert len(w) == 6 and w[0] == [1, 2, 3] and w[5] == [6, 7, 8]
    view = it.slice_windows([1, 2, 3, 4, 5], 2)
    assert len(view) == 4 and view.size_hint() == (4, 4)


def test_stream_fusion_cache_oblivious_zipper():
    assert list(it.StreamFusion([1, 2, 3, 4, 5], lambda x: x * 2 if x % 2 == 0 else None)) == [4, 8]
    r = list(it.CacheOblivious([1, 2, 3, 4, 5, 6, 7, 8], 3))
    assert len(r) == 8 and 1 in r and 8 in r
    z = it.Zipper([1, 2, 3, 4, 5])
    assert z.current() == 5
    assert z.move_right() and z.current() == 1
    assert z.move_right() and z.current() == 2
    assert z.move_right() and z.current() == 3
    assert z.move_left() and z.current() == 2
    assert z.into_vec() == [5, 1, 2, 3, 4]


def test_iterator_chain_and_batches():
    data = ["hello", "world", "from", "rust", "llm"]
    assert it.Iter(data).windows(2).map(lambda w: f"{w[0]}-{w[1]}").collect() == [
        "hello-world", "world-from", "from-rust", "rust-llm"]
    assert list(it.Iter(range(1, 10)).batch(3, 3)) == [[1, 2, 3], [4, 5, 6], [7, 8, 9]]
    b = list(it.Iter(range(1, 9)).batch(2, 4).with_memory_limit(100))
    assert len(b) == 2 and len(b[0]) == 4 and len(b[1]) == 4


def test_memory_limit_carries_item_over():
    # the reference drops the item that overflowed (iterator.rs:617-624); here nothing is lost
    b = list(it.Iter(range(10)).batch(1, 8).with_memory_limit(12))
    assert [x for batch in b for x in batch] == list(range(10))


def test_literature_iterators():
    root = it.RopeNode.Branch(it.RopeNode.Leaf("hello"), it.RopeNode.Leaf(" world"))
    assert "".join(it.RopeIterator(root)) == "hello world"
    assert "".join(it.RopeIterator(it.RopeNode.Leaf(""))) == ""
    nodes = [it.BTreeNode([1, 3]), it.BTreeNode([5, 7]), it.BTreeNode([4], [0, 1])]
    assert list(it.BTreeIterator(nodes)) == [1, 3, 4, 5, 7]
    s = list(it.SuffixArrayIterator("banana"))
    assert len(s) == 6 and s[0] == "a" and s[1] == "ana" and s[2] == "anana"
    f = it.BloomFilterBitIterator(100, 0.01)
    for i in (5, 10, 15):
        f.set_bit(i)
    bits = list(f)
    assert len(bits) == f.bit_count() and sum(bits) == f.popcount() == 3
    assert "".join(it.Iter(["hello", " ", "world"]).into_rope_owned()) == "hello world"
    assert list(it.WaveletTreeIterator([3, 1, 2])) == [1, 2, 3]
    assert list(it.TrieIterator(["dog", "cat"])) == ["cat", "dog"]


# ------------------------------------------------------------------ src/foundation/memory.rs
def test_arena_pool_cow_builder():
    arena = Arena.new(1024)
    assert arena.alloc(42) == 42
    assert bytes(arena.alloc_slice([1, 2, 3, 4, 5])) == bytes([1, 2, 3, 4, 5])
    assert arena.used() > 0
    arena.reset()
    assert arena.used() == 0
    pool = Pool.with_initializer(10, lambda: bytearray(100))
    buf = pool.take_or_init()
    assert len(buf) >= 100
    pool.put(buf)
    assert pool.len() == 1 and pool.take() is buf
    cow = CowStr.borrowed("hello")
    assert cow.is_borrowed()
    cow.push_str(" world")
    assert not cow.is_borrowed() and cow.as_str() == "hello world"
    b = ZeroCopyStringBuilder.new()
    b.append_borrowed("Hello").append_borrowed(" ").append_owned("World")
    assert b.build() == "Hello World"


def test_arena_per_thread():
    results = []

    def work(i):
        a = Arena.new(256)
        vals = [a.alloc(i * 100 + j) for j in range(50)]
        results.append(vals == [i * 100 + j for j in range(50)])

    ts = [threading.Thread(target=work, args=(i,)) for i in range(10)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert all(results) and len(results) == 10


def test_tracking_arena_bump_interner():
    t = TrackingArena.new(128)
    t.alloc_slice(b"abcdef")
    s = t.stats()
    assert s.allocation_count == 1 and s.used_bytes == 6 and s.peak_bytes == 6
    t.reset()
    assert t.stats().used_bytes == 0 and t.stats().fragmentation_ratio() == 1.0
    b = BumpAllocator.new(16)
    assert b.alloc_slice(b"12345678") is not None and b.alloc_slice(b"123456789") is None
    assert b.remaining() == 8
    si = StringInterner.new()
    a1, a2 = si.intern("tok"), si.intern("tok")
    assert a1 is a2 and si.stats().cache_hits == 1 and si.stats().memory_saved == 3 and si.len() == 1


# ------------------------------------------------------------------ src/foundation/error.rs, types.rs
def test_errors():
    ctx = ErrorContext("test_operation").at("test.rs", 42, 10).with_details("test details")
    assert ctx.operation == "test_operation" and ctx.location is not None and ctx.details == "test details"
    assert "tokenizer not initialized" in str(ProcessingError.not_initialized("tokenizer"))
    comp = CompositeError(invalid_input("bad data")).with_related(
        limit_exceeded("token", 100, 150)).with_transaction_id("tx-123")
    assert len(comp.related) == 1 and comp.transaction_id == "tx-123"
    c = error_context("macro_test")
    assert c.operation == "macro_test" and c.location is not None
    assert error_context("macro_test", "with details").details == "with details"
    assert "operation failed" in str(internal_error("test").with_context("operation failed"))
    assert str(limit_exceeded("token", 100, 150)) == "Processing error: token limit exceeded: 150 > 100"


def test_version_and_shape():
    v1, v2, v3 = Version.new(1, 0, 0), Version.new(1, 1, 0), Version.new(2, 0, 0)
    assert v2.is_compatible_with(v1) and not v1.is_compatible_with(v2) and not v1.is_compatible_with(v3)
    assert str(Version.parse("1.2.3")) == "1.2.3"
    with pytest.raises(ProcessingError):
        Version.parse("1.2")
    s1, s3 = Shape.new([2, 3, 4]), Shape.new([3, 4])
    assert s1.ndim() == 3 and s1.numel() == 24
    assert s1.is_compatible_with(Shape.new([2, 3, 4])) and not s1.is_compatible_with(s3)
    assert s1.is_compatible_with(Shape.new([2, 1, 4])) and str(Shape.new([2, 3])) == "[2, 3]"


# ------------------------------------------------------------------ src/core/config.rs
def test_config_values_builder_store():
    assert ConfigValue.of(True).as_bool() is True
    assert ConfigValue.of(42).as_integer() == 42 and ConfigValue.of(42).as_float() == 42.0
    assert ConfigValue.of(3.14).as_float() == 3.14 and ConfigValue.of("x").as_string() == "x"
    cfg = ConfigBuilder.map().with_("name", "test").with_("value", 42).with_("enabled", True).build()
    m = cfg.as_map()
    assert m["name"].as_string() == "test" and m["value"].as_integer() == 42 and m["enabled"].as_bool()
    store = ConfigStore.new()
    store.set("key1", "value1")
    store.set("key2", 42)
    assert store.get("key1").as_string() == "value1" and store.get("key2").as_integer() == 42
    assert store.get("nope") is None and store.get_or_default("nope", 7).as_integer() == 7
    other = ConfigStore.new()
    other.set("key1", "override")
    store.merge(other)
    assert store.get("key1").as_string() == "override"
    assert store.remove("key2").as_integer() == 42 and sorted(store.keys()) == ["key1"]
    pm = PluginConfigManager.new()
    pm.set_plugin_key("tokenizer", "max_length", 512)
    assert pm.get_plugin_key("tokenizer", "max_length").as_integer() == 512
    pm.set_plugin_config("tokenizer", {"a": 1})
    assert pm.get_plugin_config("tokenizer").as_map()["a"].as_integer() == 1


def test_config_layering():
    store = ConfigStore()
    store.load_mapping({"train": {"lr": 1e-3, "steps": 10}})
    store.load_env(environ={"COEUS_TRAIN__LR": "3e-4", "OTHER": "x"})
    rest = store.load_args(["--train.steps=20", "--verbose", "pos"])
    assert store.get("train.lr").as_float() == 3e-4 and store.get("train.steps").as_integer() == 20
    assert store.get("verbose").as_bool() and rest == ["pos"]


# ------------------------------------------------------------------ src/core/model.rs
def test_model_configs():
    BasicModelConfig().validate()
    with pytest.raises(ConfigError):
        BasicModelConfig(model_dim=0).validate()
    with pytest.raises(ConfigError):
        BasicModelConfig(model_dim=511).validate()
    c = Transformer250MConfig()
    assert (c.hidden_dim, c.num_layers, c.num_heads, c.intermediate_dim, c.vocab_size,
            c.max_seq_len, c.use_bias, c.activation) == (768, 12, 12, 3072, 50257, 1024, True, "gelu")
    c.validate()
    assert c.buffer_parameters() == 163_087_441 and c.num_parameters() == 163_037_184
    assert Transformer250MConfig.benchmark_250m().buffer_parameters() == 267_633_920
    for bad in (dict(hidden_dim=0), dict(hidden_dim=769), dict(num_layers=0), dict(vocab_size=0)):
        with pytest.raises(ConfigError):
            Transformer250MConfig(**bad).validate()
    msg = ""
    try:
        Transformer250MConfig(hidden_dim=769).validate()
    except ConfigError as e:
        msg = str(e)
    assert "Hidden dimension must be divisible by number of heads" in msg


def test_tensor_and_generation_config():
    t = Tensor.new(Shape.new([2, 3]), [1, 2, 3, 4, 5, 6])
    assert t.as_slice().tolist() == [1, 2, 3, 4, 5, 6]
    with pytest.raises(ProcessingError):
        Tensor.new(Shape.new([2, 3]), [1, 2, 3])
    assert Tensor.zeros(Shape.new([4])).as_slice().sum() == 0
    g = BasicGenerationConfig()
    assert (g.max_length, g.temperature, g.top_k, g.top_p) == (100, 1.0, None, None)


# ------------------------------------------------------------------ src/core/plugin.rs, plugins/*
def test_plugin_state_machine_and_capabilities():
    S = PluginState
    assert S.Registered.can_transition_to(S.Ready) and S.Ready.can_transition_to(S.Running)
    assert S.Running.can_transition_to(S.Stopped) and S.Stopped.can_transition_to(S.Running)
    assert not S.Registered.can_transition_to(S.Running) and not S.Stopped.can_transition_to(S.Ready)
    assert S.Running.can_transition_to(S.Error) and S.Error.can_transition_to(S.Registered)
    assert S.Ready.is_usable() and S.Ready.can_start() and S.Running.can_stop()
    caps = PluginCapabilities.standard().with_feature("test")
    assert caps.lifecycle and caps.has_feature("test") and not caps.has_feature("nope")
    e = PluginEntry.new(BasicTokenizerPlugin())
    with pytest.raises(PluginError):
        e.transition_to(S.Running)


def test_manager_lifecycle_and_events():
    mgr = PluginManager.new()
    seen = []
    mgr.subscribe(lambda ev: seen.append(ev.kind))
    mgr.register(BasicTokenizerPlugin)
    with pytest.raises(PluginError):
        mgr.register(BasicTokenizerPlugin)
    mgr.load("basic_tokenizer")
    with pytest.raises(PluginError):
        mgr.load("basic_tokenizer")
    assert mgr.info("basic_tokenizer").state is PluginState.Ready
    mgr.start("basic_tokenizer")
    mgr.stop("basic_tokenizer")
    assert mgr.with_plugin("basic_tokenizer", lambda p: p.id()) == "basic_tokenizer"
    mgr.unload("basic_tokenizer")
    assert seen == ["Registered", "Loaded", "Started", "Stopped", "Unloaded"]
    with pytest.raises(PluginError) as ei:
        mgr.load("missing")
    assert "not found" in str(ei.value)


def test_registry_and_builder():
    reg = PluginRegistry.new()
    reg.register(BasicTokenizerPlugin)
    assert reg.contains("basic_tokenizer") and reg.create("basic_tokenizer").id() == "basic_tokenizer"
    with pytest.raises(PluginError):
        reg.register(BasicTokenizerPlugin)
    assert reg.name_for_type(BasicTokenizerPlugin) == "basic_tokenizer"
    reg2 = (PluginRegistryBuilder.new().with_plugin(BasicTokenizerPlugin)
            .with_factory("custom", lambda: BpeTokenizerPlugin()).build())
    assert sorted(reg2.list()) == ["basic_tokenizer", "custom"]
    reg2.unregister("custom")
    assert not reg2.contains("custom")


def test_load_with_deps():
    mgr = PluginManager()
    mgr.register(BasicTokenizerPlugin)
    mgr.register(BpeTokenizerPlugin, deps=["basic_tokenizer"])
    mgr.load_with_deps("bpe_tokenizer")
    assert sorted(mgr.list_loaded()) == ["basic_tokenizer", "bpe_tokenizer"]
    assert [str(d) for d in mgr.info("bpe_tokenizer").dependencies] == ["basic_tokenizer"]


def test_concurrent_plugin_loading():
    mgr = PluginManager()
    mgr.register(BasicTokenizerPlugin)
    mgr.register(BasicModelPlugin)
    errors = []

    def work(i):
        try:
            mgr.load("basic_tokenizer" if i % 2 == 0 else "basic_model")
        except PluginError:
            errors.append(i)

    ts = [threading.Thread(target=work, args=(i,)) for i in range(10)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert len(mgr.list_loaded()) == 2 and len(errors) == 8


# ------------------------------------------------------------------ src/core/serialization.rs
def test_serialization_pieces():
    h = ModelHeader.new(Version.new(1, 0, 0), 1000, 4000)
    assert h.magic == b"RUSTLLM\x00" and h.format_version == 1 and len(h.to_bytes()) == 136
    h.validate()
    assert ModelHeader.from_bytes(h.to_bytes()).param_count == 1000
    with pytest.raises(ProcessingError):
        ModelHeader.from_bytes(b"X" * 136)
    params = [1.0, 2.0, 3.0, 4.0, 5.0]
    buf = io.BytesIO()
    assert ParameterSerializer.new().write_parameters(buf, params) == 20
    buf.seek(0)
    assert ParameterSerializer.new().read_parameters(buf, 5).tolist() == params
    md = ModelMetadata.new("transformer").with_custom("layers", "12").with_custom("heads", "8")
    md.training_config = "lr=0.001"
    back = ModelMetadata.from_bytes(md.to_bytes())
    assert back.architecture == "transformer" and back.training_config == "lr=0.001"
    assert back.custom == [("layers", "12"), ("heads", "8")]
    with pytest.raises(ProcessingError):
        ModelMetadata.from_bytes(md.to_bytes()[:7])
    assert calculate_checksum([1.0, 2.0, 3.0]) != calculate_checksum([1.0, 2.0, 3.0001])
    # the definition, element by element
    c = 0
    for x in np.array([1.5, -2.25, 3.0], dtype=np.float32):
        c = (c + int(np.float32(x).view(np.uint32))) & (2 ** 64 - 1)
        c = ((c << 1) | (c >> 63)) & (2 ** 64 - 1)
    assert calculate_checksum([1.5, -2.25, 3.0]) == c


# ------------------------------------------------------------------ src/core/tokenizer.rs, traits.rs
def test_tokens_and_tokenizer_config():
    t = StringToken.new("hello")
    assert t.as_str() == "hello" and t.id() == 0 and t.as_bytes() == b"hello" and t.len() == 5
    assert StringToken.with_id("world", 42).id() == 42
    p = PositionedToken.new(StringToken.with_id("test", 10), 5, 9)
    assert (p.as_str(), p.id(), p.start(), p.end()) == ("test", 10, 5, 9)
    c = TokenizerConfig()
    assert c.max_length is None and c.add_special_tokens and not c.lowercase
    assert c.padding is PaddingStrategy.None_ and c.truncation is TruncationStrategy.None_


def test_pipe_composition():
    class AddOne(Process):
        def id(self):
            return "add-one"

        def process(self, x):
            return x + 1

    class MultiplyTwo(Process):
        def id(self):
            return "multiply-two"

        def process(self, x):
            return x * 2

    piped = AddOne().pipe(MultiplyTwo())
    assert piped.process(5) == 12 and piped.id() == "add-one"
    assert AddOne().type_name().endswith("AddOne")


# ------------------------------------------------------------------ tokenizer plugins
def test_basic_tokenizer_roundtrip():
    tok = BasicTokenizerPlugin().create_tokenizer()
    toks = list(tok.tokenize_str("Hello, RustLLM!"))
    assert toks and tok.decode(toks).strip() == "Hello, RustLLM!" and tok.vocab_size() == 0


def test_bpe_tokenizer():
    tok = BpeTokenizerPlugin().create_tokenizer()
    assert tok.vocab_size() == 260
    toks = list(tok.tokenize_str("hello"))
    assert len(toks) == 5 and tok.decode(toks) == "hello"
    for name, i in (("<PAD>", 0), ("<UNK>", 1), ("<BOS>", 2), ("<EOS>", 3)):
        assert tok.id_from_token(name) == i and tok.token_from_id(i) == name
    before = tok.vocab_size()
    tok.train(["the cat sat on the mat", "the dog sat on the log", "the cat and the dog"], 10)
    assert tok.vocab_size() > before and tok.vocab_size() > 256
    out = tok.decode(list(tok.tokenize_str("the cat")))
    assert "the" in out and "cat" in out and out == "the cat"
    tok.add_token("custom_token")
    assert tok.contains_token("custom_token")
    tok.remove_token("custom_token")
    with pytest.raises(ProcessingError) as ei:
        tok.remove_token("custom_token")
    assert "Token not found: custom_token" in str(ei.value)
    assert [t.id() for t in tok.tokenize_str("a  b\n")] == [97, 32, 98]
    assert tok.decode_ids(tok.encode("café")) == "caf��"


def test_bpe_matches_sequential_merge_definition():
    """Native merging (rank lookup) against the reference's definition: one left-to-right pass
    per merge in learned order (plugins/tokenizer-bpe/src/lib.rs:245-271)."""
    import random
    rng = random.Random(0)
    words = ["".join(rng.choice("abcde") for _ in range(rng.randint(1, 9))) for _ in range(300)]
    tok = BpeTokenizer()
    tok.train([" ".join(words)], 40)
    merges = tok.merges()

    def ref_bpe(word):
        toks = list(word)
        for a, b in merges:
            out, i = [], 0
            while i < len(toks):
                if i + 1 < len(toks) and toks[i] == a and toks[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(toks[i])
                    i += 1
            toks = out
        return toks

    for w in words + ["abcabcabc", "eeeee", "ab"]:
        assert [t.as_str() for t in tok.tokenize_str(w)] == ref_bpe(w)


def test_wordpiece_tokenizer():
    tok = WordPieceTokenizerPlugin().create_tokenizer()
    assert tok.name() == "wordpiece"
    assert [tok.token_to_id(s) for s in ("[UNK]", "[CLS]", "[SEP]", "[PAD]", "[MASK]")] == [0, 1, 2, 3, 4]
    assert tok.token_to_id("a") == 100 and tok.token_to_id("A") == 126 and tok.token_to_id("##ing") == 152
    assert tok.normalize("café") != "café"
    toks = list(tok.tokenize_str("Hello world"))
    assert toks[0].as_str() == "[CLS]" and toks[-1].as_str() == "[SEP]"
    assert tok.decode(toks) != "" or len(toks) > 2
    assert tok.longest_match("##ing") == (152, 5)
    ids = tok.encode("testing")
    assert ids == [1, 119, 155, 152, 2]
    assert tok.decode(list(tok.tokenize_str("testing"))) == "testing"


# ------------------------------------------------------------------ model plugins, integration
def test_basic_model_and_loader():
    model = BasicModelPlugin().create_builder().build(BasicModelConfig())
    assert model.num_parameters() > 0 and model.forward([1.0, 2.0, 3.0]) == [1.0, 2.0, 3.0]
    loader = BasicLoaderPlugin()
    assert "txt" in loader.supported_formats() and "safetensors" in loader.supported_formats()
    assert loader.load_model("m.json").num_parameters() == 1000
    with pytest.raises(ProcessingError):
        loader.load_model("m.bin")


def test_integration_registration_and_iterators():
    mgr = PluginManager.new()
    for p in (BasicTokenizerPlugin, BpeTokenizerPlugin, BasicModelPlugin, BasicLoaderPlugin,
              TransformerModelPlugin, WordPieceTokenizerPlugin):
        mgr.register(p)
    avail = mgr.list_registered()
    for n in ("basic_tokenizer", "bpe_tokenizer", "basic_model", "basic_loader",
              "transformer_model", "wordpiece_tokenizer"):
        assert n in avail
    toks = list(BasicTokenizer().tokenize_str("one two three four five six seven eight nine ten"))
    assert len(it.Iter(toks).windows(3).collect()) == len(toks) - 2
    assert len(it.Iter(toks).stride(2).collect()) == (len(toks) + 1) // 2
    chunks = it.Iter(toks).chunks(2).collect()[:3]
    assert len(chunks) == 3 and len(chunks[0]) == 2


def test_concurrent_plugin_access():
    mgr = PluginManager()
    mgr.register(BasicTokenizerPlugin)
    mgr.load("basic_tokenizer")
    out = []
    ts = [threading.Thread(target=lambda: out.append(mgr.with_plugin("basic_tokenizer", lambda p: p.id())))
          for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert out == ["basic_tokenizer"] * 4


def test_prelude_exports_every_name_of_the_reference_prelude():
    """src/lib.rs:113-157: the named re-exports plus the public items behind the three glob
    re-exports (``traits::*``, ``iterator::*``, ``types::*``)."""
    import coeus_b200.prelude as P
    named = """ConfigBuilder ConfigStore ConfigValue Configurable PluginConfigManager
        BasicGenerationConfig BasicModelConfig DiffusionSampler ForwardModel GenerationConfig
        GenerativeModel Loss Model ModelBuilder ModelConfig NoiseSchedule OptimizerState
        TrainableModel Transformer250MConfig Plugin calculate_checksum ModelHeader ModelMetadata
        ModelSerializable ParameterSerializer Token Tokenizer Error Arena CowStr LazyAlloc SliceView
        ZeroCopyStringBuilder PluginManager InferenceEvent InferenceRequest InferenceResult
        InferenceService InferenceSession Architecture DomainModelAggregate ModelRepository
        ModelingEvent ModelingService DomainCheckpoint PersistenceEvent PersistenceService
        SerializationFormat StorageBackend DomainToken TokenizationEvent TokenizationService
        TokenizerAggregate TokenizerRepository Optimizer DomainTrainingConfig TrainingEvent
        TrainingService TrainingSession""".split()
    traits = """Identity Versioned Metadata Lifecycle AsyncLifecycle Process StreamProcess
        BatchProcess Serialize Checkpoint HealthCheck Metrics Validate Constraint Builder Factory
        Adapter Strategy Pipeline Piped Component ComponentInfo IntoIterator FromIterator""".split()
    iterators = """IteratorAdapter StatefulIterator PreciseSizeHint Windows SliceWindows
        StreamFusion CacheOblivious Zipper Chunks Stride BatchIterator Scan Prefetch
        ZeroCopyTokenizer ZeroCopySplit IteratorExt AdvancedIteratorExt RopeIterator
        OwnedRopeIterator BTreeIterator SuffixArrayIterator WaveletTreeIterator TrieNode
        TrieIterator BloomFilterBitIterator slice_windows slice_windows_step""".split()
    types = """Version TokenId VocabSize SequenceLength BatchSize ModelDim HeadCount LayerCount
        ModelFloat ModelDouble DynError PluginName ConfigKey Shape DType""".split()
    missing = [n for n in named + traits + iterators + types if not hasattr(P, n)]
    assert not missing, missing
    # the framework's own entry points travel with it
    for n in ("Trainer", "TrainConfig", "InferenceEngine", "ContinuousBatcher", "ParallelConfig",
              "DecoderConfig"):
        assert hasattr(P, n)
    assert P.PreciseSizeHint([1, 2, 3]).exact_size() == 3
    assert P.PreciseSizeHint(iter([1])).exact_size() is None and P.PreciseSizeHint([]).is_empty()


def test_transformer_plugin_math_helpers():
    """plugins/model-transformer/src/lib.rs:50-128 with the values its own unit tests use
    (matmul of a 2x3 by a 3x2, softmax summing to one, gelu(0) = 0, layer_norm of 1..4)."""
    import math as pymath
    import torch
    from coeus_b200.plugins.builtin import model_transformer as MT
    m = MT.math
    assert m.matmul([1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], 2, 2, 3).tolist() == [58, 64, 139, 154]
    p = m.softmax([1.0, 2.0, 3.0])
    assert abs(float(p.sum()) - 1.0) < 1e-6 and p[2] > p[1] > p[0]
    assert m.gelu(0.0) == 0.0 and abs(m.gelu(1.0) - 0.8411919906) < 1e-6
    assert abs(m.gelu(-1.0) + 0.1588080094) < 1e-6
    y = m.layer_norm([1.0, 2.0, 3.0, 4.0], [1.0] * 4, [0.0] * 4, 1e-5)
    assert abs(float(y.mean())) < 1e-6 and abs(float((y * y).mean()) - 1.0) < 1e-4
    # statistics span the whole buffer; scale and bias repeat with their own length
    x = torch.arange(12.0)
    z = m.layer_norm(x, [1.0, 2.0], [0.5], 1e-5)
    mean, var = x.mean(), ((x - x.mean()) ** 2).mean()
    want = torch.tensor([1.0, 2.0]).repeat(6) * (x - mean) / torch.sqrt(var + 1e-5) + 0.5
    assert torch.allclose(z, want, atol=1e-6)
    assert pymath.isclose(float(m.gelu(torch.tensor([2.0]))), m.gelu(2.0), rel_tol=1e-6)


def test_bpe_tokenizer_save_and_load(tmp_path):
    from coeus_b200.plugins.builtin.tokenizer_bpe import BpeTokenizer
    t = BpeTokenizer()
    t.train(["the cat sat on the mat", "naïve café 日本語", "the dog"], 50)
    path = str(tmp_path / "tok.json")
    t.save(path)
    u = BpeTokenizer.load(path)
    assert u.vocab_size() == t.vocab_size() and u.merges() == t.merges()
    for s in ("the cat sat", "café 日本 xyz", "  spaced   out "):
        assert u.encode(s).tolist() == t.encode(s).tolist()
        assert u.decode_ids(u.encode(s)) == t.decode_ids(t.encode(s))


def test_wordpiece_tokenizer_save_and_load(tmp_path):
    from coeus_b200.plugins.builtin.tokenizer_wordpiece import WordPieceTokenizer
    t = WordPieceTokenizer()
    for i, tok in enumerate(["un", "##aff", "##able", "caf", "##é", "日本"]):
        t.add_token(tok, 5000 + i)
    path = str(tmp_path / "wp.json")
    t.save(path)
    u = WordPieceTokenizer.load(path)
    assert u.vocab_size() == t.vocab_size() and u.vocabulary() == t.vocabulary()
    for s in ("unaffable café", "hello 日本 world"):
        assert u.encode(s) == t.encode(s)
