"""The benchmark's own construction path on CPU: the configuration ``bench.py`` builds must
validate, a model must come out of it, and one whole training step must run through the same
``build_arm`` the timed run uses (one layer and a short batch keep it quick)."""
import dataclasses
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_every_preset_validates():
    from coeus_b200.models.config import DecoderConfig, Transformer250MConfig
    for cfg in (DecoderConfig.transformer_250m(), DecoderConfig.decoder_1p3b(),
                DecoderConfig.moe_8x()):
        cfg.validate()
    Transformer250MConfig().validate()
    Transformer250MConfig.benchmark_250m().validate()
    # the preset of the benchmark keeps the reference's fields and trains without dropout
    cfg = DecoderConfig.transformer_250m(max_seq_len=2048)
    assert (cfg.hidden_dim, cfg.num_layers, cfg.num_heads, cfg.intermediate_dim,
            cfg.vocab_size, cfg.max_seq_len) == (1024, 16, 16, 4096, 32000, 2048)
    assert cfg.dropout == 0.0 and cfg.attention_dropout == 0.0


def test_bench_config_builds_and_trains_on_cpu():
    import bench
    cfg = bench.build_config(64)
    cfg.validate()
    small = dataclasses.replace(cfg, num_layers=1)
    step, par, owner = bench.build_arm("coeus", small, torch.device("cpu"), 1)
    assert par == "single GPU"
    batch = torch.randint(0, small.vocab_size, (1, 17))
    l0 = float(step(batch))
    l1 = float(step(batch))
    assert l0 > 0 and l1 < l0


def test_bench_torch_arm_builds_on_cpu():
    import bench
    small = dataclasses.replace(bench.build_config(64), num_layers=1)
    from coeus_b200.models.torch_baseline import TorchDecoder
    m = TorchDecoder(small, torch.device("cpu"))
    batch = torch.randint(0, small.vocab_size, (1, 17))
    loss = m(batch[:, :-1], batch[:, 1:])
    loss.backward()
    assert torch.isfinite(loss)


def test_reference_probe_is_a_run_time_probe():
    import bench
    probe = bench.probe_reference_toolchain()
    assert set(probe) == {"rustc", "cargo", "ref_installed"}


@pytest.mark.timeout(600)
def test_cpu_baseline_script_runs():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "cpu_baseline.py"),
                        "--skip-oracle", "--layers", "1", "--steps", "1"],
                       capture_output=True, text=True, timeout=580)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["torch_cpu_train"]["tokens_per_s"] > 0 and out["bpe_1mb"]["roundtrip_exact"]
