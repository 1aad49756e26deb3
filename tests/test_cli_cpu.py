"""``python -m coeus_b200``: layered configuration, training (one process and two Gloo ranks under
torchrun), saving, generating from the saved file."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = ["--device=cpu", "--model.hidden_dim=32", "--model.num_layers=2", "--model.num_heads=2",
         "--model.intermediate_dim=64", "--model.vocab_size=320", "--model.max_seq_len=32",
         "--train.seq_len=16", "--train.batch=4", "--train.lr=0.01", "--train.log_every=100"]


def _run(args, env=None, launcher=None, timeout=600):
    cmd = [sys.executable] + (launcher or []) + ["-m", "coeus_b200"] + args
    e = {**os.environ, **(env or {})}
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT, env=e)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return json.loads([l for l in r.stdout.strip().splitlines() if l.startswith("{")][-1])


def test_layering_file_env_args(tmp_path):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("model:\n  hidden_dim: 64\n  num_heads: 2\ntrain:\n  lr: 0.5\n")
    out = _run(["info", str(cfg), "--model.num_layers=3"], env={"COEUS_TRAIN__LR": "0.25"})
    assert out["model"]["hidden_dim"] == 64 and out["model"]["num_layers"] == 3
    assert out["config"]["train.lr"] == 0.25        # environment over file, arguments over both
    assert out["parameters"] > 0


def test_train_on_text_save_and_generate(tmp_path):
    text = tmp_path / "corpus.txt"
    text.write_text("\n".join(["the cat sat on the mat", "the dog sat on the log"] * 60))
    weights = tmp_path / "m.safetensors"
    metrics = tmp_path / "metrics.jsonl"
    out = _run(["train"] + SMALL + ["--train.steps=12", f"--data.files={text}",
                                    f"--train.save={weights}", "--train.warmup=2",
                                    f"--train.metrics_file={metrics}"])
    assert out["strategy"] == "single" and out["steps"] == 12
    events = [json.loads(l) for l in metrics.read_text().splitlines()]
    assert events[0]["event"] == "TrainingEvent::Started"
    steps_logged = [e for e in events if e["event"] == "TrainingEvent::StepCompleted"]
    assert [e["step"] for e in steps_logged] == list(range(1, 13)) and steps_logged[0]["tokens"] == 64
    assert out["last_loss"] < out["first_loss"]
    gen = _run(["generate", "--device=cpu", f"--weights={weights}", "--prompt_ids=5,6,7",
                "--max_tokens=4"])
    assert gen["prompt_ids"] == [5, 6, 7] and len(gen["token_ids"]) == 4
    # the tokenizer was saved beside the weights: text in, text out
    assert os.path.exists(str(weights) + ".tokenizer.json")
    gen = _run(["generate", "--device=cpu", f"--weights={weights}", "--prompt=the cat",
                "--max_tokens=3"])
    assert len(gen["prompt_ids"]) >= 1 and isinstance(gen["text"], str)
    ev = _run(["eval", "--device=cpu", f"--weights={weights}", f"--data.files={text}",
               "--train.seq_len=16", "--train.batch=4", "--max_batches=5"])
    assert ev["tokens"] == 5 * 4 * 16 and ev["loss"] < out["first_loss"]
    assert abs(ev["perplexity"] - __import__("math").exp(ev["loss"])) < 1e-3 * ev["perplexity"]


def test_train_two_ranks_under_torchrun(tmp_path):
    import socket
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    launcher = ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                "--master-addr=127.0.0.1", f"--master-port={port}"]
    text = tmp_path / "corpus.txt"
    text.write_text("\n".join(["the cat sat on the mat", "the dog sat on the log"] * 60))
    out = _run(["train"] + SMALL + ["--train.steps=12", "--parallel.dp=2", f"--data.files={text}",
                                    f"--train.checkpoint_dir={tmp_path}/ck",
                                    "--train.checkpoint_every=6"], launcher=launcher)
    assert out["strategy"] == "dp" and out["world"] == 2 and out["last_loss"] < out["first_loss"]
    assert os.path.exists(tmp_path / "ck" / "manifest.json")


def test_injected_fault_then_resume_matches_the_uninterrupted_run(tmp_path):
    """A host-side fault after step 7 kills the run; the restart picks up the step-5 checkpoint
    and ends where the uninterrupted run ends."""
    text = tmp_path / "corpus.txt"
    text.write_text("\n".join(["the cat sat on the mat", "the dog sat on the log",
                               "a cat and a dog and a mat"] * 80))
    common = SMALL + [f"--data.files={text}", "--train.checkpoint_every=5", "--train.steps=10"]
    whole = _run(["train"] + common + [f"--train.checkpoint_dir={tmp_path}/a"])
    env = {**os.environ, "PYTHONPATH": ROOT + os.pathsep + os.environ.get("PYTHONPATH", "")}
    crash = subprocess.run([sys.executable, "-m", "coeus_b200", "train"] + common +
                           [f"--train.checkpoint_dir={tmp_path}/b", "--train.fault=after_step:7"],
                           capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert crash.returncode != 0 and "after_step" in crash.stderr
    rest = _run(["train"] + common + [f"--train.checkpoint_dir={tmp_path}/b",
                                      "--train.resume=true"])
    assert rest["resumed_at"] == 5 and abs(rest["last_loss"] - whole["last_loss"]) < 1e-5
