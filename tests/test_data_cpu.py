"""Host side of the input pipeline (no GPU): ordering with worker threads, epochs, resume from
state_dict, sharding, the token-window dataset, error delivery."""
import time

import numpy as np
import pytest

from mytorch_b200.utils.data import DataLoader, Dataset, TokenLoader


class Squares(Dataset):
    def __init__(self, n, delay=False):
        self.n, self.delay = n, delay

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if self.delay:
            time.sleep(0.002 * ((i * 7) % 5))     # workers finish out of order
        return np.array([i, i * i]), np.float32(i)


@pytest.mark.parametrize("workers", [0, 3])
def test_batches_arrive_in_order_and_epochs_advance(workers):
    dl = DataLoader(Squares(23, delay=True), batch_size=4, num_workers=workers)
    assert len(dl) == 6
    for epoch in range(2):
        got = [b for b in dl]
        assert len(got) == 6 and got[-1][0].shape == (3, 2)
        flat = np.concatenate([b[0][:, 0] for b in got])
        assert np.array_equal(flat, np.arange(23))
        assert np.array_equal(np.concatenate([b[1] for b in got]), np.arange(23, dtype=np.float32))
        assert dl.epoch == epoch + 1 and dl.batches_consumed == 0
    dl.shutdown()


def test_resume_from_state_dict_continues_the_same_shuffled_epoch():
    np.random.seed(3)
    dl = DataLoader(Squares(40), batch_size=4, shuffle=True, num_workers=2)
    it = iter(dl)
    first = [next(it)[0][:, 0].copy() for _ in range(3)]
    state = dl.state_dict()
    rest = []
    while True:          # `for b in it` would call __iter__ again and restart the epoch
        try:
            rest.append(next(it)[0][:, 0].copy())
        except StopIteration:
            break
    assert state["batches_consumed"] == 3 and len(state["shuffled_indices"]) == 40
    dl2 = DataLoader(Squares(40), batch_size=4, shuffle=True, num_workers=2)
    dl2.load_state_dict(state)
    rest2 = [b[0][:, 0].copy() for b in dl2]
    assert len(rest2) == len(rest) == 7
    assert all(np.array_equal(a, b) for a, b in zip(rest, rest2))
    assert sorted(np.concatenate(first + rest).tolist()) == list(range(40))


def test_worker_exception_reaches_the_consumer():
    class Bad(Squares):
        def __getitem__(self, i):
            if i == 9:
                raise ValueError("sample 9 is broken")
            return super().__getitem__(i)

    dl = DataLoader(Bad(16), batch_size=4, num_workers=2)
    it = iter(dl)
    next(it); next(it)
    with pytest.raises(ValueError, match="sample 9"):
        next(it)
    dl.shutdown()


def test_shard_interleaves_indices_across_ranks():
    base = DataLoader(Squares(16), batch_size=4)
    seen = []
    for rank in range(2):
        seen.append(np.concatenate([b[0][:, 0] for b in base.shard(rank, 2)]))
    assert np.array_equal(seen[0], np.arange(0, 16, 2)) and np.array_equal(seen[1], np.arange(1, 16, 2))


def test_token_loader_windows_are_shifted_by_one_and_reproducible():
    toks = np.random.default_rng(0).integers(0, 50257, 5000).astype(np.uint16)
    a, b = TokenLoader(toks, 64, seed=1, rank=0), TokenLoader(toks, 64, seed=1, rank=1)
    x, y = a[5]
    assert x.dtype == np.uint16 and x.shape == (64,) and np.array_equal(x[1:], y[:-1])
    x2, _ = TokenLoader(toks, 64, seed=1, rank=0)[5]
    assert np.array_equal(x, x2)
    assert not np.array_equal(x, b[5][0])
    xb, yb = next(iter(DataLoader(a, batch_size=8, num_workers=2)))
    assert xb.shape == yb.shape == (8, 64)
