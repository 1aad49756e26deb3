"""Tracing, metrics, health and events on CPU."""
import json

import torch

from coeus_b200.utils.metrics import (EventBus, JsonlSink, TrainerMonitor, device_memory_stats,
                                      model_flops_per_token)
from coeus_b200.utils.tracing import PhaseTimer, nvtx_range


def _trainer():
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cfg = DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    return Trainer(DecoderLM(cfg, "cpu", seed=1, dtype=torch.float32), TrainConfig(learning_rate=1e-2))


def test_phase_timer_and_nvtx_are_usable_without_a_gpu():
    t = PhaseTimer("cpu")
    with nvtx_range("outer"):
        with t.phase("a"):
            sum(range(1000))
        with t.phase("a"):
            pass
        with t.phase("b"):
            pass
    s = t.summary()
    assert set(s) == {"a", "b"} and s["a"] >= 0 and t.counts() == {"a": 2, "b": 1}
    assert t.summary() == {}


def test_monitor_metrics_health_and_events(tmp_path):
    tr = _trainer()
    bus = EventBus()
    seen = []
    bus.subscribe(seen.append)
    sink = JsonlSink(str(tmp_path / "events.jsonl"))
    bus.subscribe(sink)
    mon = TrainerMonitor(tr, seq_len=16, peak_tflops=1.0, bus=bus)
    def batches():
        g = torch.Generator().manual_seed(0)       # the same three batches every epoch
        for _ in range(3):
            b = torch.randint(0, 64, (2, 17), generator=g)
            yield b[:, :-1].contiguous(), b[:, 1:].contiguous()

    mon.fit(batches, epochs=2)
    sink.close()
    kinds = [e["event"] for e in seen]
    assert kinds == ["TrainingEvent::Started", "TrainingEvent::EpochCompleted",
                     "TrainingEvent::EpochCompleted"]
    m = {x.name: x.value for x in mon.metrics()}
    assert m["steps"] == 6 and m["tokens"] == 6 * 32 and m["tokens_per_s"] > 0 and m["mfu"] > 0
    assert seen[2]["mean_loss"] < seen[1]["mean_loss"]          # it learns the repeated stream
    assert mon.health().healthy
    lines = [json.loads(l) for l in open(tmp_path / "events.jsonl")]
    assert len(lines) == 3
    mon.reset_metrics()
    assert {x.name: x.value for x in mon.metrics()}["steps"] == 0


def test_flops_model_and_memory_stats_shape():
    from coeus_b200.models.config import DecoderConfig
    cfg = DecoderConfig.transformer_250m()
    f = model_flops_per_token(cfg, 2048, True)
    n_matrix = 16 * (4 * 1024 * 1024 + 2 * 1024 * 4096) + 1024 * 32000
    assert f > 6 * n_matrix and f < 8 * n_matrix
    st = device_memory_stats("cpu")
    assert st.used_bytes == 0 and st.fragmentation_ratio() == 0.0


def test_rank_prefixed_logging():
    import io
    import logging
    from coeus_b200.utils.logging import get_logger, log_sink, setup_logging
    buf = io.StringIO()
    setup_logging(logging.INFO, rank=0, world=8, stream=buf)
    get_logger("train").info("step %d", 3)
    log_sink({"event": "TrainingEvent::Started"})
    out = buf.getvalue()
    assert "[rank 0/8] INFO coeus_b200.train: step 3" in out and "TrainingEvent::Started" in out
    buf = io.StringIO()
    setup_logging(logging.INFO, rank=5, world=8, stream=buf)       # other ranks: problems only
    get_logger("train").info("quiet")
    get_logger("train").warning("loud")
    assert "quiet" not in buf.getvalue() and "[rank 5/8] WARNING" in buf.getvalue()
    buf = io.StringIO()
    setup_logging(logging.INFO, rank=5, world=8, all_ranks=True, stream=buf)
    get_logger().info("everyone")
    assert "everyone" in buf.getvalue()


def test_per_op_ranges_wrap_every_kernel_entry_point(monkeypatch):
    from coeus_b200.ops import _lib

    class Fake:
        def __init__(self):
            self.calls = []

        def cb_gemm(self, a, b):
            self.calls.append(("gemm", a, b))
            return 0

        def cb_fails(self):
            raise RuntimeError("boom")

        other = staticmethod(lambda: 7)

    fake = Fake()
    monkeypatch.setattr(_lib, "_lib", fake)
    log = []
    _lib.set_op_ranges(True, push=lambda n: log.append(("push", n)), pop=lambda: log.append(("pop",)))
    try:
        assert _lib.lib().cb_gemm(1, 2) == 0 and _lib.lib().cb_gemm(3, 4) == 0
        assert _lib.lib().other() == 7                       # not an op: not wrapped
        try:
            _lib.lib().cb_fails()
        except RuntimeError:
            pass
        assert log == [("push", "cb_gemm"), ("pop",), ("push", "cb_gemm"), ("pop",),
                       ("push", "cb_fails"), ("pop",)]       # the range closes on errors too
        assert fake.calls == [("gemm", 1, 2), ("gemm", 3, 4)]
    finally:
        _lib.set_op_ranges(False)
    assert _lib.lib() is fake
