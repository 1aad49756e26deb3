"""The parts of the benchmark's contract that need no GPU: the reference arm's one-line answer,
the flags, and the shape of the JSON line (from the source, since the timed arms need a B200)."""
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str)
    assert "\n" not in line["unavailable"] and len(line["unavailable"]) > 20


def test_json_line_has_every_contract_key():
    src = open(os.path.join(ROOT, "bench.py")).read()
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config",
                "clocks", "gpu_launches", "e2e", "h2d_bytes_per_step", "d2h_bytes_per_step",
                "global_batch", "seq_len", "parallelism", "model"):
        assert re.search(rf'"{key}"', src), key
    # defaults finish quickly on one GPU; at least three warm-up steps are enforced
    assert 'add_argument("--gpus", type=int, default=1)' in src
    assert "args.warmup = max(args.warmup, 3)" in src
    # the metric is the one the baseline file names
    base = json.load(open(os.path.join(ROOT, "BASELINE.json")))
    metric = re.search(r'METRIC = "([^"]+)"', src).group(1)
    assert "tokens/s" in metric or "tokens/sec" in metric
    assert "token" in json.dumps(base).lower()


def test_multi_gpu_request_without_launcher_is_refused_cleanly():
    env = {k: v for k, v in os.environ.items() if k not in ("WORLD_SIZE", "RANK", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"],
                       capture_output=True, text=True, timeout=300, env=env)
    # either the clean refusal (no launcher) or, on a box without CUDA, a CUDA error before it
    assert r.returncode != 0


def test_packaging_metadata_points_at_real_files():
    import glob
    import tomllib
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        meta = tomllib.load(f)
    assert meta["project"]["name"] == "coeus_b200"
    mod, fn = meta["project"]["scripts"]["coeus"].split(":")
    assert callable(getattr(__import__(mod, fromlist=[fn]), fn))
    for pattern in meta["tool"]["setuptools"]["package-data"]["coeus_b200"]:
        assert glob.glob(os.path.join(ROOT, "coeus_b200", pattern)), pattern
