"""Every example program runs on CPU and produces what it says."""
import importlib.util
import os

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _load(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(ROOT, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_basic_usage():
    r = _load("basic_usage").main()
    assert r["decoded"].strip() == "Hello, RustLLM Core! This is a simple example."
    assert r["trigrams"] == r["tokens"] - 2 and r["cow"] == "hello world" and r["built"] == "zero-copy"
    assert r["loaded"] == ["basic_tokenizer"] and r["arena_used"] > 0


def test_config_usage():
    r = _load("config_usage").main(["--verbose", "positional"])
    assert r == {"layers": 24, "lr": 1e-4, "steps": 200, "vocab": 50000, "name": "example",
                 "rest": ["positional"]}


def test_streaming():
    r = _load("streaming").main(lines=500, sentences=30)
    assert r["stream_tokens"] > 500 * 10 and r["windows3"] == 7 and r["windows5"] == 5
    assert r["bpe_tokens"] > 0 and r["top"]


def test_training_example():
    r = _load("training_example").main(["--device", "cpu", "--steps", "12"])
    assert r["toy"][-1] < r["toy"][0] * 0.5
    assert r["lm"][-1] < r["lm"][0]


def test_transformer_example_small():
    r = _load("transformer_250m").main(["--small", "--device", "cpu"])
    assert r["logits"] == 320 and r["roundtrip_identical"] and len(r["generated"]) == 8
    assert r["file_bytes"] > 136 + 4 * r["params"] and r["loaded"] == ["transformer_model"]


def test_diffusion_example():
    r = _load("diffusion_example").main(40)
    assert r["end_mse"] < r["start_mse"] * 0.25 and r["deterministic"] and r["view_len"] == 16
    assert 0 < r["alpha_bar_last"] < 1


def test_wordpiece_example():
    r = _load("wordpiece_tokenizer").main(5)
    assert r["pieces"]["unaffable"] == ["[CLS]", "un", "##aff", "##able", "[SEP]"]
    assert r["pieces"]["playing played"][1:-1] == ["play", "##ing", "play", "##ed"]
    assert "[UNK]" in r["pieces"]["xylophone"]
    assert r["chars_per_s"] > 0


def test_serve_completions_dry_run():
    assert _load("serve_completions").main(["--device", "cpu", "--dry-run"]) == 0


def test_serving_benchmark_runs_small():
    spec = importlib.util.spec_from_file_location(
        "bench_serving", os.path.join(os.path.dirname(ROOT), "benchmarks", "serving.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    r = mod.main(["--device", "cpu", "--requests", "5", "--max-seqs", "2", "--hidden", "64",
                  "--layers", "2", "--heads", "2", "--prompt-max", "24", "--new-max", "6"])
    assert r["generated_tokens"] > 0 and r["batched_tokens_per_s"] > 0
    assert r["latency_s"]["p50"] <= r["latency_s"]["max"]


def test_parallel_training_example_single_process():
    r = _load("parallel_training").main(["--device", "cpu", "--steps", "6"])
    assert r["strategy"] == "single" and r["last"] < r["first"]


def test_autograd_training_example():
    r = _load("autograd_training").main(["--device", "cpu", "--steps", "25"])
    assert r["last"] < 0.6 * r["first"] and r["grad_norm"] > 0


def _load_bench(name):
    spec = importlib.util.spec_from_file_location(
        f"bench_{name}", os.path.join(os.path.dirname(ROOT), "benchmarks", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_tokenizer_and_iterator_microbenchmarks_run():
    """Counterparts of the reference's criterion benches (benches/tokenizer_bench.rs,
    benches/iterator_bench.rs, benches/advanced_iterator_bench.rs, wordpiece_bench.rs)."""
    t = _load_bench("tokenizer_bench").main()
    assert t["bpe/tokenize/lorem"] > 0 and any(k.startswith("wordpiece/encode") for k in t)
    it = _load_bench("iterator_bench").main()
    assert it["windows/5"] > 0 and "prefetch/64" in it and "rolling_average" in it
