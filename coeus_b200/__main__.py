"""Command line: ``python -m coeus_b200 <command> [config files] [--key=value ...]``.

Commands
    train      build a model and a trainer from the layered configuration and train it
    generate   load a model file and continue a prompt
    eval       load a model file and report loss / perplexity on text or token files
    serve      load a model file (or build a random one) and serve completions over HTTP
    info       print the resolved configuration and the parameter count

Configuration comes, lowest priority first, from the built-in defaults, the given ``.yaml`` /
``.json`` files, ``COEUS_*`` environment variables (``COEUS_TRAIN__LR=1e-4`` sets ``train.lr``)
and ``--key=value`` arguments (``--train.lr=1e-4``).  Under ``torchrun`` the process group is
initialised from the environment (NCCL on GPUs, Gloo on CPU) and ``parallel.*`` selects the
strategy.  The reference stops at a config store with no file, environment or command-line
front end ("Implement configuration system" is unchecked in its CHECKLIST.md:64).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Any, Dict, List, Optional

DEFAULTS: Dict[str, Any] = {
    "model": {"preset": "", "hidden_dim": 256, "num_layers": 4, "num_heads": 4, "num_kv_heads": 0,
              "intermediate_dim": 1024, "vocab_size": 512, "max_seq_len": 256, "use_bias": False,
              "activation": "swiglu", "norm": "rmsnorm", "pos": "rope", "recompute": False},
    "parallel": {"dp": 1, "tp": 1, "pp": 1, "ep": 1, "cp": 1, "ulysses": False,
                 "micro_batches": 1, "pp_chunks": 1, "zero_stage": 2},
    "train": {"steps": 20, "batch": 4, "seq_len": 128, "lr": 3e-4, "warmup": 0, "grad_clip": 0.0,
              "weight_decay": 0.01, "seed": 0, "log_every": 5, "checkpoint_dir": "",
              "checkpoint_every": 0, "save": "", "resume": False, "watchdog": True,
              "fault": "", "metrics_file": ""},
    "data": {"files": "", "binary": "", "binary_dtype": "uint16"},
    "device": "auto",
}


def _resolve(argv: List[str]):
    from .core.config import ConfigStore
    store = ConfigStore()
    store.load_mapping(DEFAULTS)
    rest = []
    for a in argv:
        if a.endswith((".yaml", ".yml", ".json")) and not a.startswith("--"):
            store.load_file(a)
        else:
            rest.append(a)
    store.load_env()
    rest = store.load_args(rest)
    return store, rest


def _get(store, key: str):
    v = store.get(key)
    if v is None:
        return None
    for conv in (v.as_bool, v.as_integer, v.as_float, v.as_string):
        try:
            out = conv()
        except Exception:
            out = None
        if out is not None:
            return out
    return None


def _model_config(store):
    from .models.config import DecoderConfig
    preset = _get(store, "model.preset") or ""
    if preset:
        make = {"250m": DecoderConfig.transformer_250m, "1.3b": DecoderConfig.decoder_1p3b,
                "moe": DecoderConfig.moe_8x}.get(str(preset).lower())
        if make is None:
            raise SystemExit(f"unknown model.preset '{preset}' (250m, 1.3b, moe)")
        return make()
    keys = ("hidden_dim", "num_layers", "num_heads", "num_kv_heads", "intermediate_dim", "vocab_size",
            "max_seq_len", "use_bias", "activation", "norm", "pos")
    return DecoderConfig(**{k: _get(store, f"model.{k}") for k in keys})


def _device(store) -> str:
    import torch
    d = _get(store, "device")
    if d in (None, "auto"):
        return "cuda" if torch.cuda.is_available() else "cpu"
    return str(d)


def _init_distributed(device: str):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        return 0, 1, device
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if device.startswith("cuda"):
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        device = f"cuda:{local}"
        dist.init_process_group("nccl", device_id=torch.device(device))
    else:
        dist.init_process_group("gloo")
    return dist.get_rank(), world, device


def cmd_train(store) -> dict:
    import numpy as np
    import torch

    from .core.config import ParallelConfig
    from .optim.lr import Constant, WarmupCosine
    from .train.data import TokenDataset
    from .train.launch import build_trainer
    from .train.trainer import TrainConfig
    from .utils.logging import setup_logging
    device = _device(store)
    rank, world, device = _init_distributed(device)
    log = setup_logging(rank=rank, world=world)
    cfg = _model_config(store)
    par = ParallelConfig(**{k: _get(store, f"parallel.{k}")
                            for k in ("dp", "tp", "pp", "ep", "cp", "pp_chunks", "zero_stage")},
                         ulysses=bool(_get(store, "parallel.ulysses")))
    steps, B, S = (_get(store, f"train.{k}") for k in ("steps", "batch", "seq_len"))
    lr, warm = _get(store, "train.lr"), _get(store, "train.warmup")
    clip = _get(store, "train.grad_clip") or None
    tc = TrainConfig(learning_rate=lr, weight_decay=_get(store, "train.weight_decay"),
                     grad_clip=clip)
    sched = WarmupCosine(lr, warm, steps, floor=0.1 * lr) if warm else Constant(lr)
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    run = build_trainer(cfg, par, device, tc, micro_batches=_get(store, "parallel.micro_batches"),
                        seed=_get(store, "train.seed"), dtype=dtype,
                        recompute=bool(_get(store, "model.recompute")), schedule=sched)
    # data: text files through a byte-level BPE tokenizer, a binary token file, or random ids
    files, binary = _get(store, "data.files"), _get(store, "data.binary")
    if binary:
        ds = TokenDataset.from_binary(binary, S, B, dtype=np.dtype(_get(store, "data.binary_dtype")))
    elif files:
        from .prelude import BpeTokenizerPlugin
        tok = BpeTokenizerPlugin().create_tokenizer()
        paths = [p for p in str(files).split(",") if p]
        with open(paths[0], encoding="utf-8", errors="replace") as f:
            tok.train(f.read(1 << 20).splitlines(), max(0, cfg.vocab_size - 300))
        ds = TokenDataset.from_text_files(paths, tok, S, B)
        if _get(store, "train.save") and rank == 0:     # the tokenizer travels with the model
            tok.save(str(_get(store, "train.save")) + ".tokenizer.json")
    else:
        g = np.random.default_rng(_get(store, "train.seed"))
        ds = TokenDataset(g.integers(0, cfg.vocab_size, size=(steps + 1) * B * S + 1), S, B)
    ckpt_dir, every = _get(store, "train.checkpoint_dir"), _get(store, "train.checkpoint_every")
    losses, step, epoch = [], 0, 0
    skip = 0
    if _get(store, "train.resume") and ckpt_dir and hasattr(run.trainer, "load_checkpoint") \
            and os.path.exists(os.path.join(ckpt_dir, "manifest.json")):
        meta = run.trainer.load_checkpoint(ckpt_dir)
        meta = meta.get("meta", meta)
        step = int(meta.get("train_step", 0))
        per_epoch = max(1, ds.num_windows() // B)
        epoch, skip = divmod(step, per_epoch)       # continue inside the epoch that was running
        log.info("resumed from %s at step %d (epoch %d, batch %d)", ckpt_dir, step, epoch, skip)
    resumed_at = step
    from .parallel.health import FaultInjector, StepWatchdog
    import time as _time
    watchdog = StepWatchdog() if _get(store, "train.watchdog") else None
    # host-side fault injection for resume drills: --train.fault=after_step:7 raises there
    injector = FaultInjector(str(_get(store, "train.fault") or "") or None)
    slow = 0
    from .utils.metrics import EventBus, JsonlSink, model_flops_per_token
    bus = EventBus()
    if _get(store, "train.metrics_file") and rank == 0:      # one JSON line per step
        bus.subscribe(JsonlSink(str(_get(store, "train.metrics_file"))))
    bus.emit("TrainingEvent::Started", strategy=run.strategy, world=world, resumed_at=step)
    flops_tok = model_flops_per_token(cfg, S, True)
    t_run, tok_run = _time.perf_counter(), 0
    t_log, tok_log = t_run, 0
    while step < steps:
        ds.reset(epoch)
        if skip:
            ds.seek(skip)
            skip = 0
        got = False
        for ids, tgt in ds:
            got = True
            ids, tgt = ids.to(device), tgt.to(device)
            t_step = _time.perf_counter()
            loss = float(run.step(ids, tgt))
            losses.append(loss)
            step += 1
            if watchdog is not None and watchdog.observe(_time.perf_counter() - t_step):
                slow += 1
                log.warning("step %d took %.3f s, far above the recent median", step,
                            _time.perf_counter() - t_step)
            injector.reach("after_step")
            tok_run += ids.numel()
            tok_log += ids.numel()
            bus.emit("TrainingEvent::StepCompleted", step=step, loss=loss,
                     seconds=_time.perf_counter() - t_step, tokens=ids.numel())
            if step % max(1, _get(store, "train.log_every")) == 0:
                now = _time.perf_counter()      # float(loss) above already waited for the device
                tps = tok_log / max(now - t_log, 1e-9)
                log.info("step %d loss %.4f  %.0f tokens/s  %.2f TFLOP/s", step, loss, tps,
                         tps * flops_tok / 1e12)
                t_log, tok_log = now, 0
            if ckpt_dir and every and step % every == 0 and hasattr(run.trainer, "save_checkpoint"):
                run.trainer.save_checkpoint(ckpt_dir)
            if step >= steps:
                break
        if not got:
            raise SystemExit("the data source yields no full batch")
        epoch += 1
    save = _get(store, "train.save")
    if save and run.strategy in ("single", "dp", "cp"):
        dp = getattr(run.trainer, "dp", None)
        if dp is not None:
            run.model.p32.copy_(dp.gather_master())
        if rank == 0:
            from .checkpoint.formats import save_model
            save_model(run.model, save)
    elif save and run.strategy in ("tp", "dp+tp"):
        run.model.save(save)
    out = {"strategy": run.strategy, "steps": step, "resumed_at": resumed_at,
           "first_loss": losses[0] if losses else None,
           "last_loss": losses[-1] if losses else None, "world": world, "slow_steps": slow,
           "tokens_per_s": tok_run / max(_time.perf_counter() - t_run, 1e-9)}
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return out


def _load_weights(weights: str, device: str, training: bool = False):
    """A model file (``.safetensors`` / ``.gguf`` / ``.rustllm``) or a Hugging Face style
    directory (``config.json`` + ``*.safetensors``, Llama naming)."""
    if os.path.isdir(weights):
        from .checkpoint.hf import load_hf_dir
        return load_hf_dir(weights, device=device, training=training)
    from .checkpoint.formats import load_model
    return load_model(weights, device=device, training=training)[0]


def _load_tokenizer(store, weights: str):
    """``--tokenizer=file`` or the file the training command wrote beside the weights."""
    path = _get(store, "tokenizer") or (weights + ".tokenizer.json" if weights else None)
    # a Hugging Face model directory brings its own tokenizer files
    hf_dir = str(_get(store, "tokenizer") or weights or "")
    if os.path.isdir(hf_dir) and any(os.path.exists(os.path.join(hf_dir, f))
                                     for f in ("tokenizer.json", "tokenizer.model")):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(hf_dir)
    if not path or not os.path.exists(str(path)):
        return None
    from .plugins.builtin.tokenizer_bpe import BpeTokenizer
    return BpeTokenizer.load(str(path))


def cmd_generate(store, rest: List[str]) -> dict:
    import torch

    from .infer.engine import InferenceEngine
    device = _device(store)
    weights = _get(store, "weights")
    if not weights:
        raise SystemExit("generate needs --weights=<file.safetensors|.gguf|.rustllm>")
    model = _load_weights(str(weights), device)
    tok = _load_tokenizer(store, str(weights))
    ids_arg, text = _get(store, "prompt_ids"), _get(store, "prompt")
    if ids_arg is not None:
        ids = [int(t) for t in str(ids_arg).split(",")]
    elif text is not None and tok is not None:
        ids = [int(t) for t in tok.encode(str(text))]
    else:
        raise SystemExit("generate needs --prompt_ids=1,2,3, or --prompt=text with a tokenizer "
                         "file (<weights>.tokenizer.json or --tokenizer=...)")
    n = int(_get(store, "max_tokens") or 16)
    out = InferenceEngine(model, max_batch=1).generate(
        torch.tensor(ids, device=device)[None], n,
        temperature=float(_get(store, "temperature") or 0.0))
    res = {"prompt_ids": ids, "token_ids": out[0, len(ids):].tolist()}
    if tok is not None:
        from .serve.server import _decoder
        res["text"] = _decoder(tok)(res["token_ids"])
    print(json.dumps(res))
    return res


def cmd_eval(store) -> dict:
    import numpy as np

    from .train.data import TokenDataset
    from .train.trainer import Trainer
    device = _device(store)
    weights = _get(store, "weights")
    if not weights:
        raise SystemExit("eval needs --weights=<file>")
    model = _load_weights(str(weights), device, training=True)
    S = min(int(_get(store, "train.seq_len")), model.cfg.max_seq_len)
    B = int(_get(store, "train.batch"))
    files, binary = _get(store, "data.files"), _get(store, "data.binary")
    if binary:
        ds = TokenDataset.from_binary(str(binary), S, B,
                                      dtype=np.dtype(_get(store, "data.binary_dtype")))
    elif files:
        tok = _load_tokenizer(store, str(weights))
        if tok is None:
            raise SystemExit("eval on text needs the tokenizer (<weights>.tokenizer.json or "
                             "--tokenizer=...)")
        ds = TokenDataset.from_text_files([p for p in str(files).split(",") if p], tok, S, B)
    else:
        raise SystemExit("eval needs --data.files=... or --data.binary=...")
    limit = int(_get(store, "max_batches") or 0)

    def batches():
        for i, (ids, tgt) in enumerate(ds):
            if limit and i >= limit:
                return
            yield ids.to(device), tgt.to(device)
    out = Trainer(model).evaluate(batches())
    print(json.dumps(out))
    return out


def cmd_serve(store) -> int:
    """One process: a single-GPU engine behind HTTP.  Under ``torchrun`` the ranks form one
    tensor-parallel group: every rank holds its shards and runs the serving loop, rank 0 also
    runs the HTTP server and feeds the others."""
    import torch

    from .models.decoder import DecoderLM
    from .serve import ServingLoop, create_app
    device = _device(store)
    rank, world, device = _init_distributed(device)
    weights = _get(store, "weights")
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    if weights:
        model = _load_weights(str(weights), device if world == 1 else "cpu")
    else:
        model = DecoderLM(_model_config(store), device if world == 1 else "cpu",
                          dtype=dtype if world == 1 else torch.float32, training=False)
    max_seqs = int(_get(store, "max_seqs") or 16)
    kw = dict(max_seqs=max_seqs, max_len=model.cfg.max_seq_len)
    engine = group = None
    if world > 1:
        import torch.distributed as dist

        from .infer.tp_engine import TPInferenceEngine
        from .parallel.tp import TensorParallel
        from .parallel.tp_model import TPDecoderLM
        group = dist.group.WORLD
        tpm = TPDecoderLM(model.cfg, TensorParallel(group, device), device, dtype=dtype, full=model)
        engine = TPInferenceEngine(tpm, max_batch=max_seqs, use_graph=False)
        if rank != 0:
            loop = ServingLoop(None, engine=engine, group=group, **kw)
            loop.join()
            return 0
    import uvicorn
    app = create_app(model, tokenizer=_load_tokenizer(store, str(weights) if weights else ""),
                     prefix_cache=bool(_get(store, "prefix_cache")), engine=engine, group=group,
                     **kw)
    uvicorn.run(app, host=str(_get(store, "host") or "127.0.0.1"),
                port=int(_get(store, "port") or 8000))
    return 0


def cmd_info(store) -> dict:
    from .models.decoder import ParamLayout
    cfg = _model_config(store)
    out = {"model": cfg.to_dict(), "parameters": ParamLayout(cfg).num_parameters(),
           "config": {k: _get(store, k) for k in sorted(store.keys())}}
    print(json.dumps(out))
    return out


def main(argv: Optional[List[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    cmd, store_rest = argv[0], _resolve(argv[1:])
    store, rest = store_rest
    if cmd == "train":
        return cmd_train(store)
    if cmd == "generate":
        return cmd_generate(store, rest)
    if cmd == "eval":
        return cmd_eval(store)
    if cmd == "serve":
        return cmd_serve(store)
    if cmd == "info":
        return cmd_info(store)
    raise SystemExit(f"unknown command '{cmd}' (train, generate, eval, serve, info)")


if __name__ == "__main__":
    r = main()
    sys.exit(r if isinstance(r, int) else 0)
