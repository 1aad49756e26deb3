"""Training checkpoints keyed by tensor name, for models whose ranks hold different tensors
(pipeline stages) or different rows of the same tensors (expert shards).

Every rank writes one SafeTensors file with the fp32 master weights and the two Adam moments of
the tensors it holds (``w/<name>``, ``m/<name>``, ``v/<name>``); tensors sharded over experts
carry the index of their first global row in the file's metadata.  Loading asks for tensors by
name (and row range) and finds them in whichever files hold them, so a run resumes with another
number of pipeline stages or another expert-parallel degree.  The reference's ``Checkpoint``
entity has an id and an epoch and nothing behind it (src/domain/persistence/mod.rs:10-29).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Callable, Dict, Optional, Tuple

import torch

from ..foundation.error import ProcessingError
from ..utils import native
from .formats import _load_indexed, save_safetensors

STATE_KEYS = ("w", "m", "v")


def model_state(model, opt) -> Dict[str, Tuple[Dict[str, torch.Tensor], int]]:
    """``name -> ({"w","m","v"} tensors, first global row)`` of a :class:`DecoderLM` (possibly a
    pipeline stage or an expert shard) and its AdamW state over the same flat layout."""
    out = {}
    ep_rank = model.epx.rank if model.epx is not None else 0
    for s in model.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        row0 = ep_rank * s.shape[0] if (s.expert and model.layout.ep > 1) else 0
        out[s.name] = ({"w": model.p32[sl].view(s.shape), "m": opt.m[sl].view(s.shape),
                        "v": opt.v[sl].view(s.shape)}, row0)
    return out


def save_named(directory: str, rank: int, state, meta: dict,
               barrier: Optional[Callable[[], None]] = None) -> None:
    os.makedirs(directory, exist_ok=True)
    if barrier is not None:
        barrier()
    tensors, rows = {}, {}
    for name, (parts, row0) in state.items():
        for k in STATE_KEYS:
            tensors[f"{k}/{name}"] = parts[k]
        rows[name] = row0
    save_safetensors(os.path.join(directory, f"part{rank}.safetensors"), tensors,
                     {"rows": json.dumps(rows)})
    if barrier is not None:
        barrier()
    if rank == 0:
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump({"kind": "named", **meta}, f)
    if barrier is not None:
        barrier()


def load_named(directory: str, state) -> dict:
    """Fill the tensors of ``state`` (as from :func:`model_state`) from the files of
    ``directory``; returns the manifest."""
    with open(os.path.join(directory, "manifest.json")) as f:
        man = json.load(f)
    if man.get("kind") != "named":
        raise ProcessingError.invalid_input(f"{directory} is not a name-keyed checkpoint")
    files = []
    for path in sorted(glob.glob(os.path.join(directory, "part*.safetensors"))):
        index = native.module().safetensors_index(path)
        rows = json.loads(dict(index["metadata"]).get("rows", "{}"))
        have = {t["name"]: t for t in index["tensors"]}
        files.append((path, index, rows, have))
    for name, (parts, row0) in state.items():
        want_rows = parts["w"].shape[0] if parts["w"].dim() > 0 else 1
        filled = 0
        for path, index, rows, have in files:
            if f"w/{name}" not in have:
                continue
            f_row0 = int(rows.get(name, 0))
            f_rows = have[f"w/{name}"]["shape"][0] if have[f"w/{name}"]["shape"] else 1
            lo, hi = max(row0, f_row0), min(row0 + want_rows, f_row0 + f_rows)
            whole = f_row0 == 0 and row0 == 0 and f_rows == want_rows
            if not whole and hi <= lo:
                continue
            got = _load_indexed(path, index, names={f"{k}/{name}" for k in STATE_KEYS})
            for k in STATE_KEYS:
                src = got[f"{k}/{name}"]
                if whole:
                    parts[k].copy_(src)
                else:
                    parts[k][lo - row0:hi - row0].copy_(src[lo - f_row0:hi - f_row0])
            if whole:
                filled = want_rows
                break
            filled += hi - lo
        if filled < want_rows:
            raise ProcessingError.invalid_input(
                f"checkpoint {directory} holds {filled} of {want_rows} rows of '{name}'")
    return man
