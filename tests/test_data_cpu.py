"""Token dataset over the native batch loader and the prefetcher (CPU path)."""
import numpy as np
import pytest
import torch

from coeus_b200.train.data import DevicePrefetcher, TokenDataset


def test_windows_targets_and_rank_split():
    toks = np.arange(1000, dtype=np.int32)
    ds = TokenDataset(toks, seq_len=9, batch=4, stride=9)
    batches = list(ds)
    x, y = batches[0]
    assert x.shape == (4, 9) and torch.equal(y, x + 1)          # next-token targets
    assert x[0, 0] == 0 and x[1, 0] == 9                        # consecutive windows
    assert len(batches) == ds.num_windows() // 4
    ds.reset()
    r0 = [b[0] for b in TokenDataset(toks, 9, 4, rank=0, world=2)]
    r1 = [b[0] for b in TokenDataset(toks, 9, 4, rank=1, world=2)]
    assert torch.equal(r0[0], batches[0][0]) and torch.equal(r1[0], batches[1][0])
    assert abs(len(r0) - len(r1)) <= 1


def test_shuffle_is_seeded_and_seek_resumes():
    toks = np.arange(2000, dtype=np.int32)
    a = [b[0] for b in TokenDataset(toks, 15, 4, shuffle=True, seed=3)]
    b = [b[0] for b in TokenDataset(toks, 15, 4, shuffle=True, seed=3)]
    c = [b[0] for b in TokenDataset(toks, 15, 4, shuffle=True, seed=4)]
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert any(not torch.equal(x, y) for x, y in zip(a, c))
    ds = TokenDataset(toks, 15, 4, shuffle=True, seed=3)
    it = iter(ds)
    next(it); next(it)
    cur = ds.cursor()
    assert cur == 2
    ds2 = TokenDataset(toks, 15, 4, shuffle=True, seed=3)
    ds2.seek(cur)
    rest = [b[0] for b in ds2]
    assert len(rest) == len(a) - 2 and all(torch.equal(x, y) for x, y in zip(rest, a[2:]))


def test_prefetcher_passes_batches_through_on_cpu():
    toks = np.arange(500, dtype=np.int32)
    want = [b[0] for b in TokenDataset(toks, 9, 2)]
    got = [b[0] for b in DevicePrefetcher(TokenDataset(toks, 9, 2), "cpu")]
    assert len(want) == len(got) and all(torch.equal(a, b) for a, b in zip(want, got))


def test_dataset_from_text_files_and_binary(tmp_path):
    import numpy as np
    from coeus_b200.prelude import BpeTokenizerPlugin
    from coeus_b200.train.data import TokenDataset, save_tokens, tokenize_files
    tok = BpeTokenizerPlugin().create_tokenizer()
    lines = ["the cat sat on the mat", "", "the dog sat on the log", "a cat and a dog"] * 20
    tok.train([l for l in lines if l], 30)
    a, b = tmp_path / "a.txt", tmp_path / "b.txt"
    a.write_text("\n".join(lines[:40]) + "\n")
    b.write_text("\n".join(lines[40:]))
    stream = tokenize_files([str(a), str(b)], tok, eos_id=3)
    want = []
    for l in lines:
        if l:
            want += [int(t) for t in tok.encode(l)] + [3]
    assert stream.dtype == np.int32 and stream.tolist() == want
    ds = TokenDataset.from_text_files([str(a), str(b)], tok, seq_len=16, batch=4, eos_id=3)
    ids, tgt = next(iter(ds))
    assert ids.shape == (4, 16) and torch.equal(ids[:, 1:], tgt[:, :-1])
    assert ids[0].tolist() == want[:16]
    path = tmp_path / "tokens.bin"
    save_tokens(str(path), stream)
    ds2 = TokenDataset.from_binary(str(path), seq_len=16, batch=4)
    ids2, _ = next(iter(ds2))
    assert torch.equal(ids, ids2) and ds2.num_windows() == ds.num_windows()
    with pytest.raises(ValueError):
        save_tokens(str(path), [70000], dtype=np.uint16)
