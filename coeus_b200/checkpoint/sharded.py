"""Sharded training checkpoints that can be resumed on a different number of ranks.

Every rank writes one SafeTensors file with the pieces of the flat fp32 master weights and Adam
moments it owns; a piece is named by its offset in the flat buffer (``p32@<start>``, ``m@<start>``,
``v@<start>``), so the files do not depend on how many ranks wrote them.  A JSON manifest lists the
pieces of every file with an xxhash64 of the file, the step, the world size, the model config, the
host RNG states and the data cursor.  Loading asks for arbitrary ``[start, end)`` ranges and
assembles each from whichever files overlap it (memory-mapped reads).  Saving can run in the
background: the pieces are copied to pinned host memory on a side stream and a writer thread
does the file IO.  A file whose hash no longer matches the manifest is reported as corrupt.

A save never touches the files of the previous checkpoint: every step's files carry the step in
their name and are written under a temporary name first, the manifest is replaced atomically
once all of them exist, and only then are the files that the new manifest no longer lists
removed.  A crash at any point of a save leaves the previous manifest and its files intact, so
a resume loads the last complete checkpoint.

The reference has only whole-model ``.rustllm`` files without optimizer state, and names a
``Checkpoint{checkpoint(), restore()}`` trait that nothing implements (src/core/traits.rs:181-189,
src/domain/persistence/mod.rs:10-29)."""
from __future__ import annotations

import json
import os
import threading
from typing import Callable, Dict, Optional, Sequence, Tuple

import numpy as np
import torch

from ..foundation.error import IoError, ProcessingError
from ..utils import native
from .formats import load_safetensors, save_safetensors

MANIFEST = "manifest.json"
STATE_NAMES = ("p32", "m", "v")
Segment = Tuple[int, int]

# Host-side fault injection (coeus_b200.parallel.health.FaultInjector or None): the save path
# reports the points "checkpoint.shard_written" and "checkpoint.before_manifest" to it, which is
# how the crash-during-save drill interrupts a save between the shard files and the manifest.
fault_injector = None


def _reach(point: str) -> None:
    if fault_injector is not None:
        fault_injector.reach(point)


def _shard_file(rank: int, step: int) -> str:
    return f"shard_{rank:05d}.step{step:09d}.safetensors"


def file_hash(path: str) -> str:
    """xxhash64 of a file's bytes (hex)."""
    with open(path, "rb") as f:
        data = f.read()
    return f"{native.module().xxhash64(data, 0):016x}"


class AsyncWriter:
    """At most one checkpoint in flight: ``submit`` returns at once, ``wait`` joins the thread and
    re-raises what it raised."""

    def __init__(self) -> None:
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    def submit(self, fn: Callable[[], None]) -> None:
        self.wait()

        def run():
            try:
                fn()
            except BaseException as e:   # surfaced by wait()
                self._error = e
        self._thread = threading.Thread(target=run, name="checkpoint-writer", daemon=True)
        self._thread.start()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            e, self._error = self._error, None
            raise e


def save_shard(directory: str, rank: int, world: int, segments: Sequence[Segment],
               fetch: Callable[[str, int, int], torch.Tensor], step: int,
               meta: Optional[dict] = None, writer: Optional[AsyncWriter] = None,
               barrier: Optional[Callable[[], None]] = None) -> None:
    """Write this rank's file and (rank 0, after ``barrier``) the manifest.

    ``fetch(name, start, end)`` returns the fp32 tensor of state ``name`` for the flat range.
    With ``writer`` the device-to-host copies are enqueued now and the files are written by the
    writer's thread; the manifest is then written by whoever calls :func:`finalize_manifest`."""
    os.makedirs(directory, exist_ok=True)
    host: Dict[str, torch.Tensor] = {}
    cuda_dev = None
    for s, e in segments:
        if e <= s:
            continue
        for name in STATE_NAMES:
            t = fetch(name, s, e)
            if t.is_cuda:
                cuda_dev = t.device
                buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                buf.copy_(t, non_blocking=True)
            else:
                buf = t.detach().clone()
            host[f"{name}@{s}"] = buf
    event = None
    if cuda_dev is not None:
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(cuda_dev))
    path = os.path.join(directory, _shard_file(rank, step))
    side = {"rank": rank, "world": world, "step": step,
            "segments": [[int(s), int(e)] for s, e in segments if e > s]}

    def write():
        if event is not None:
            event.synchronize()
        save_safetensors(path + ".tmp", host, {"step": str(step), "rank": str(rank)})
        side["hash"] = file_hash(path + ".tmp")
        os.replace(path + ".tmp", path)
        with open(path + ".json.tmp", "w") as f:
            json.dump(side, f)
        os.replace(path + ".json.tmp", path + ".json")

    if writer is not None:
        writer.submit(write)
        return
    write()
    _reach("checkpoint.shard_written")
    if barrier is not None:
        barrier()
    if rank == 0:
        _reach("checkpoint.before_manifest")
        finalize_manifest(directory, world, step, meta or {})
    if barrier is not None:
        barrier()


def finalize_manifest(directory: str, world: int, step: int, meta: dict) -> None:
    """Merge the per-rank side files into ``manifest.json`` (call once all files are written)."""
    files = []
    for r in range(world):
        p = os.path.join(directory, _shard_file(r, step) + ".json")
        if not os.path.exists(p):
            raise IoError.file_system(p, "open", "file not found")
        with open(p) as f:
            side = json.load(f)
        if side["step"] != step:
            raise ProcessingError.invalid_input(
                f"shard {r} is from step {side['step']}, expected {step}")
        files.append({"file": _shard_file(r, step), "segments": side["segments"], "hash": side["hash"]})
    man = {"format": "coeus-sharded-1", "step": step, "world": world, "files": files, "meta": meta}
    tmp = os.path.join(directory, MANIFEST + ".tmp")
    with open(tmp, "w") as f:
        json.dump(man, f)
    os.replace(tmp, os.path.join(directory, MANIFEST))     # atomic: a manifest is never partial
    _remove_stale_shards(directory, {e["file"] for e in files})


def _remove_stale_shards(directory: str, keep: set) -> None:
    """Delete shard files (and their side files, and left-over temporaries) that the current
    manifest does not list: the previous checkpoint's, and the remains of an interrupted save."""
    for name in os.listdir(directory):
        if not name.startswith("shard_"):
            continue
        base = name
        for suffix in (".json.tmp", ".tmp", ".json"):
            if base.endswith(suffix):
                base = base[: -len(suffix)]
                break
        if base not in keep:
            try:
                os.remove(os.path.join(directory, name))
            except OSError:
                pass


def read_manifest(directory: str) -> dict:
    p = os.path.join(directory, MANIFEST)
    if not os.path.exists(p):
        raise IoError.file_system(p, "open", "file not found")
    with open(p) as f:
        return json.load(f)


def load_ranges(directory: str, segments: Sequence[Segment],
                store: Callable[[str, int, int, torch.Tensor], None],
                verify: bool = True, state_names: Sequence[str] = STATE_NAMES) -> dict:
    """For every requested ``[start, end)`` call ``store(name, start', end', tensor)`` with the
    overlapping pieces found in the checkpoint (possibly several per range).  Returns the
    manifest."""
    man = read_manifest(directory)
    wanted = [(int(s), int(e)) for s, e in segments if e > s]
    covered = 0
    for entry in man["files"]:
        hits = []
        for fs, fe in entry["segments"]:
            for s, e in wanted:
                lo, hi = max(fs, s), min(fe, e)
                if hi > lo:
                    hits.append((fs, lo, hi))
        if not hits:
            continue
        path = os.path.join(directory, entry["file"])
        if not os.path.exists(path):
            raise IoError.file_system(path, "open", "file not found")
        if verify and file_hash(path) != entry["hash"]:
            raise IoError.file_system(path, "verify", "checksum mismatch: xxhash64 differs from the manifest")
        names = [f"{n}@{fs}" for fs in sorted({h[0] for h in hits}) for n in state_names]
        tensors, _ = load_safetensors(path, names=names)
        for fs, lo, hi in hits:
            for n in state_names:
                store(n, lo, hi, tensors[f"{n}@{fs}"][lo - fs:hi - fs])
            covered += hi - lo
    need = sum(e - s for s, e in wanted)
    if covered != need:
        raise IoError.file_system(directory, "load", f"checkpoint covers {covered} of {need} requested elements")
    return man
