"""Seeded random batches against the CPU oracle: vocabulary sizes on both sides of every path
boundary, per-row options drawn from the values that switch code paths (greedy, no cut, top-k at
1 / small / beyond the candidate buffer, top-p at 0 / inside / 1, min-p), penalties of either sign
over histories of random lengths, and both draws.  Ids, survivor counts and cuts must equal the
oracle's except on rows the oracle marks as within 1e-4 of a flipped float comparison."""

import os

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu

VOCABS = [777, 5000, 16384, 32772, 65536, 151936]
CASES = int(os.environ.get("LEAT_RANDOM_CASES", "24"))  # a longer soak: LEAT_RANDOM_CASES=400


@pytest.fixture(scope="module")
def sampler(device):
    from leat_b200.sampler import Sampler

    return Sampler(16, 262144, 256, device)


def _case(seed):
    from leat_b200 import workloads

    rng = np.random.default_rng(1000 + seed)
    vocab = VOCABS[seed % len(VOCABS)]
    rows = int(rng.integers(1, 13))
    logits = (rng.standard_normal((rows, vocab)) * rng.uniform(0.5, 5.0)).astype(np.float32)
    heavy = rng.random((rows, vocab)) < 0.002
    logits[heavy] += rng.uniform(3.0, 12.0, int(heavy.sum())).astype(np.float32)
    options = np.zeros((rows, 5), np.float32)
    options[:, 0] = np.where(rng.random(rows) < 0.2, 0.0, rng.uniform(0.3, 1.5, rows))
    options[:, 1] = rng.choice([0, 1, 5, 50, 200, 300], rows)
    options[:, 2] = rng.choice([1.0, 0.9, 0.5, 0.0], rows)
    options[:, 3] = rng.choice([0.0, 0.0, 0.02, 0.3], rows)
    history = penalties = None
    if seed % 3:
        cap = int(rng.choice([8, 100, 700]))
        history = rng.integers(0, vocab, (rows, cap)).astype(np.int32)
        best = np.argsort(-logits, axis=1)[:, : min(6, cap)]
        history[:, : best.shape[1]] = best
        penalties = np.stack([rng.choice([1.0, 1.2, 0.9], rows), rng.choice([0.0, 0.6, -0.3], rows),
                              rng.choice([0.0, 0.2], rows)], axis=1).astype(np.float32)  # fmt: skip
    return workloads.Workload(f"random{seed}", logits, options, penalties, history, rng.random(rows, dtype=np.float32),
                              rng.integers(0, 2**32, rows, dtype=np.uint64).astype(np.uint32),
                              rng.integers(0, 4096, rows).astype(np.int32))  # fmt: skip


@pytest.mark.parametrize("seed", range(CASES))
@pytest.mark.parametrize("mode", ["U", "G"])
def test_random_batch(sampler, device, seed, mode):
    import torch

    w = _case(seed)
    got = helpers.gpu_run(sampler, w, mode, device, width=0)
    want = helpers.oracle_run(w, mode, order="sequential")
    torch.cuda.synchronize()
    assert int(got.status.item()) & 4 == 0
    ids, kept, cut = got.ids.cpu().numpy().ravel(), got.kept.cpu().numpy(), got.cut.cpu().numpy()
    np.testing.assert_array_equal(got.greedy.cpu().numpy(), want.greedy)
    soft = 0
    for b in range(w.rows):
        greedy_row = not w.options[b, 0] > 0
        same = greedy_row or (kept[b] == want.kept[b] and (cut[b] == want.cut[b] or (np.isneginf(cut[b]) and np.isneginf(want.cut[b]))))
        if not (ids[b] == want.ids[b, 0] and same):
            assert want.margin[b] < 1e-4, (seed, b, w.options[b], ids[b], want.ids[b, 0], kept[b], want.kept[b], cut[b], want.cut[b], want.margin[b])
            soft += 1
    assert soft <= 2


@pytest.mark.parametrize("rows, vocab", [(130, 65536), (200, 100352), (300, 151936), (600, 70000)])
@pytest.mark.parametrize("mode", ["U", "G"])
def test_random_large_batch(device, rows, vocab, mode):
    """The same mix of options on batches of more rows than SMs, where the floors' samples are loaded
    a line per instruction, the list finish runs in its narrow blocks and, from about 440 rows on,
    the filter's blocks work the floors out themselves."""
    import torch

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler

    rng = np.random.default_rng(rows + vocab)
    logits = (rng.standard_normal((rows, vocab)) * rng.uniform(1.0, 4.0)).astype(np.float32)
    heavy = rng.random((rows, vocab)) < 0.002
    logits[heavy] += rng.uniform(3.0, 12.0, int(heavy.sum())).astype(np.float32)
    options = np.zeros((rows, 5), np.float32)
    options[:, 0] = np.where(rng.random(rows) < 0.2, 0.0, rng.uniform(0.3, 1.5, rows))
    options[:, 1] = rng.choice([1, 5, 50, 200], rows)
    options[:, 2] = rng.choice([1.0, 0.9, 0.5], rows)
    options[:, 3] = rng.choice([0.0, 0.0, 0.02], rows)
    history = rng.integers(0, vocab, (rows, 64)).astype(np.int32)
    history[:, :4] = np.argsort(-logits, axis=1)[:, :4]
    penalties = np.stack([rng.choice([1.0, 1.2], rows), rng.choice([0.0, 0.6], rows), np.zeros(rows)], axis=1).astype(np.float32)
    w = workloads.Workload("large", logits, options, penalties, history, rng.random(rows, dtype=np.float32),
                           rng.integers(0, 2**32, rows, dtype=np.uint64).astype(np.uint32),
                           rng.integers(0, 4096, rows).astype(np.int32))  # fmt: skip
    sampler = Sampler(rows, vocab, 256, device)
    got = helpers.gpu_run(sampler, w, mode, device, width=0)
    want = helpers.oracle_run(w, mode)
    helpers.compare(want, got, 0, max_fragile=3)
    np.testing.assert_array_equal(got.kept.cpu().numpy()[want.margin >= helpers.FRAGILE][options[want.margin >= helpers.FRAGILE, 0] > 0],
                                  want.kept[want.margin >= helpers.FRAGILE][options[want.margin >= helpers.FRAGILE, 0] > 0])  # fmt: skip
