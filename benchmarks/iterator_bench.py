#!/usr/bin/env python
"""Iterator and memory-utility micro-benchmarks with the workloads of the reference's
benches/iterator_bench.rs and benches/advanced_iterator_bench.rs: windows of 2/5/10 over 1000
integers, chunks, stride over 10k, zero-copy split, chained adapters, map, batch against plain
slicing, rolling average (scan), prefetch depths 16..128 against no prefetch, string builder
against ``+=`` and ``format``, lazy slice views against eager copies.  Prints nanoseconds per
operation as one JSON object."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.foundation import iterator as it
from coeus_b200.prelude import Iter, SliceView, ZeroCopyStringBuilder


def ns_per_op(fn, min_time: float = 0.05) -> float:
    fn()
    n, t = 0, 0.0
    t0 = time.perf_counter()
    while t < min_time:
        fn()
        n += 1
        t = time.perf_counter() - t0
    return t / n * 1e9


def _rolling(state, x):
    state[0] += x
    state[1] += 1
    return state, state[0] / state[1]


def main() -> dict:
    out = {}
    d1k, d10k = list(range(1000)), list(range(10_000))
    for w in (2, 5, 10):
        out[f"windows/{w}"] = ns_per_op(lambda: Iter(d1k).windows(w).collect())
        out[f"slice_windows/{w}"] = ns_per_op(lambda: sum(1 for _ in it.slice_windows(d1k, w)))
    for c in (10, 100):
        out[f"chunks/{c}"] = ns_per_op(lambda: Iter(d1k).chunks(c).collect())
    for s in (2, 10):
        out[f"stride/{s}"] = ns_per_op(lambda: Iter(d10k).stride(s).collect())
    text = ",".join(str(i) for i in range(1000))
    out["zero_copy_split"] = ns_per_op(lambda: sum(1 for _ in it.ZeroCopySplit(text, ",")))
    out["str_split"] = ns_per_op(lambda: len(text.split(",")))
    out["chained"] = ns_per_op(
        lambda: Iter(d1k).windows(3).map(lambda w: w[0] + w[1] + w[2]).stride(2).collect())
    out["map"] = ns_per_op(lambda: Iter(d1k).map(lambda x: x * 2).collect())
    out["batch/64"] = ns_per_op(lambda: sum(1 for _ in Iter(d10k).batch(64, 64)))
    out["plain_slices/64"] = ns_per_op(lambda: [d10k[i:i + 64] for i in range(0, 10_000, 64)])
    out["rolling_average"] = ns_per_op(
        lambda: Iter(d1k).scan_with([0.0, 0], _rolling).collect())
    out["no_prefetch"] = ns_per_op(lambda: sum(1 for _ in iter(d10k)))
    for depth in (16, 32, 64, 128):
        out[f"prefetch/{depth}"] = ns_per_op(lambda: Iter(d10k).prefetch(depth).collect())
    parts = [f"part{i}" for i in range(100)]

    def builder():
        b = ZeroCopyStringBuilder.new()
        for p in parts:
            b.append_borrowed(p)
        return b.build()

    def plus_eq():
        s = ""
        for p in parts:
            s += p
        return s

    out["string_builder"] = ns_per_op(builder)
    out["string_plus_eq"] = ns_per_op(plus_eq)
    out["string_format"] = ns_per_op(lambda: "".join(f"{p}" for p in parts))
    view = SliceView.new(d10k)
    out["slice_view_lazy"] = ns_per_op(lambda: len(view))
    out["slice_copy_eager"] = ns_per_op(lambda: len(list(d10k)))
    out = {k: round(v, 1) for k, v in out.items()}
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
