"""Property tests (hypothesis) of the native host components: tokenizer round trips on arbitrary
text, the token-window loader's coverage, the sharded-checkpoint range algebra."""
import re

import numpy as np
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from coeus_b200.plugins.builtin.tokenizer_bpe import BpeTokenizer

_TOK = None
# Unicode White_Space, what Rust's ``char::is_whitespace`` (and the native tokenizers) split on;
# Python's ``str.split()`` also splits on the separators U+001C..U+001F, which are not in the set
_WS = re.compile("[\t\n\x0b\x0c\r \x85\xa0\u1680\u2000-\u200a\u2028\u2029\u202f\u205f\u3000]+")


def _collapse(text: str) -> str:
    return " ".join(w for w in _WS.split(text) if w)


def _tok():
    global _TOK
    if _TOK is None:
        _TOK = BpeTokenizer()
        _TOK.train(["the cat sat on the mat", "naïve café 日本語 Ünïcödé", "a b c d e f g"], 80)
    return _TOK


@settings(max_examples=200, deadline=None)
@given(st.text(alphabet=st.characters(blacklist_categories=("Cs",)), max_size=80))
def test_bpe_lossless_round_trip_collapses_whitespace_only(text):
    """With the bytes joined before decoding, decode(encode(s)) is s with every whitespace run
    replaced by one space and the ends trimmed (words are split on whitespace and joined by the
    space token, plugins/tokenizer-bpe/src/lib.rs:284-342), for any text."""
    t = _tok()
    ids = t.encode(text)
    assert t.decode_ids(ids, ref_compat=False) == _collapse(text)
    toks = list(t.tokenize(text))                 # ids and strings stay in step
    assert [tk.id() for tk in toks] == [int(i) for i in ids]


@settings(max_examples=100, deadline=None)
@given(st.text(alphabet=st.characters(min_codepoint=9, max_codepoint=126,
                                      ),
               max_size=80))
def test_bpe_reference_decoding_round_trips_ascii(text):
    """The reference's per-byte lossy decoding is exact on ASCII; above it, unmerged bytes turn
    into U+FFFD (kept as the default for parity)."""
    t = _tok()
    assert t.decode_ids(t.encode(text)) == _collapse(text)


def test_bpe_reference_decoding_is_lossy_above_ascii():
    t = _tok()
    ids = t.encode("\x80")
    assert t.decode_ids(ids) == "\ufffd\ufffd" and t.decode_ids(ids, ref_compat=False) == "\x80"


@settings(max_examples=60, deadline=None)
@given(st.integers(30, 400), st.integers(2, 17), st.integers(1, 20), st.integers(1, 5),
       st.booleans(), st.booleans())
def test_token_loader_yields_every_window_once(n, window, step, batch, shuffle, drop_last):
    from coeus_b200.utils import native
    toks = np.arange(n, dtype=np.int32)
    ld = native.module().TokenBatchLoader(toks, window, step, batch, 2, shuffle, 5, drop_last)
    starts = list(range(0, n - window + 1, step))
    ld.reset(0)
    buf = np.empty((batch, window), dtype=np.int64)
    seen = []
    while True:
        k = ld.next_into(buf)
        if k == 0:
            break
        for r in range(k):
            row = buf[r]
            assert (np.diff(row) == 1).all()
            seen.append(int(row[0]))
    want = len(starts) - (len(starts) % batch if drop_last else 0)
    assert len(seen) == want and len(set(seen)) == len(seen) and set(seen) <= set(starts)
    if not shuffle:
        assert seen == starts[:want]


@settings(max_examples=100, deadline=None)
@given(st.integers(1, 8), st.integers(1, 8), st.integers(8, 4000))
def test_bucket_shards_tile_the_bucket_for_any_world(world_a, world_b, n8):
    """Shards of a bucket under two different world sizes both tile it exactly, which is what lets
    a checkpoint written by one world size be read by another."""
    from coeus_b200.parallel.plans import Bucket
    b = Bucket(0, 64, 64 + n8 * 8, 0, "x")
    for world in (world_a, world_b):
        pos = b.start
        for r in range(world):
            s, e = b.shard(r, world)
            assert s == pos or (s == e == b.end)
            assert (s - b.start) % 8 == 0
            pos = max(pos, e)
        assert pos == b.end


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 6), st.integers(0, 3), st.lists(st.integers(1, 300), min_size=1, max_size=12))
def test_offset_allocator_never_overlaps(align_pow, seed, sizes):
    from coeus_b200.parallel.symm import OffsetAllocator
    a = OffsetAllocator(1 << 16, alignment=1 << (align_pow + 3))
    rng = np.random.default_rng(seed)
    live = {}
    for n in sizes:
        off = a.alloc(n)
        assert off % a.alignment == 0
        for o, m in live.items():
            assert off + n <= o or o + m <= off
        live[off] = n
        if live and rng.random() < 0.4:
            victim = list(live)[int(rng.integers(len(live)))]
            a.release(victim)
            del live[victim]
    for o in list(live):
        a.release(o)
    assert a.free == [[0, 1 << 16]]
