"""Token dataset over the native batch loader and the prefetcher (CPU path)."""
import numpy as np
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
