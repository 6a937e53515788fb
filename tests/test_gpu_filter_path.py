"""The filter path (a floor per row guessed from a sample, one streaming filter, finish from the
row's list) against the CPU oracle, on inputs built to defeat the guess: rows whose large logits
all sit where the sample never looks (the list overflows), rows whose large logits all sit where
the sample does look (too few candidates above the floor), penalties that raise logits, frequency
penalties (counts, not just membership), history tokens at the top of the row, -inf logits.  Rows
the list cannot settle must come out exact through the multi-pass routine, with
LEAT_STATUS_FALLBACK set; results must not depend on whether the filter path is on."""

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu

V = 65536  # the floor kernel samples 128 logits at every multiple of 1024 here


@pytest.fixture(scope="module")
def sampler(device):
    from leat_b200.sampler import Sampler

    return Sampler(64, 262144, 256, device)


def _workload(logits, options, history=None, penalties=None, seed=7):
    from leat_b200 import workloads

    rows = logits.shape[0]
    rng = np.random.default_rng(seed)
    return workloads.Workload("case", logits, options, penalties, history, rng.random(rows, dtype=np.float32),
                              np.arange(rows, dtype=np.uint32) + 11, np.full(rows, 3, np.int32))  # fmt: skip


def _check(sampler, device, w, mode="U", expect_fallback=None, max_fragile=1):
    import torch

    want = helpers.oracle_run(w, mode, order="sequential" if expect_fallback else "block")
    got = helpers.gpu_run(sampler, w, mode, device, width=0)
    torch.cuda.synchronize()
    status = int(got.status.item())
    assert status & 4 == 0
    if expect_fallback is not None:
        assert bool(status & 1) == expect_fallback
    ids, kept, cut = got.ids.cpu().numpy().ravel(), got.kept.cpu().numpy(), got.cut.cpu().numpy()
    np.testing.assert_array_equal(got.greedy.cpu().numpy(), want.greedy)
    soft = 0
    for b in range(len(ids)):
        greedy_row = not w.options[b, 0] > 0  # no cut is defined for a greedy row
        ok = ids[b] == want.ids[b, 0] and (greedy_row or (kept[b] == want.kept[b] and cut[b] == want.cut[b]))
        if not ok:
            assert want.margin[b] < 1e-4, (b, ids[b], want.ids[b, 0], kept[b], want.kept[b], cut[b], want.cut[b])
            soft += 1
    assert soft <= max_fragile
    return got


def _options(rows, temperature=0.8, top_k=40, top_p=0.9):
    return np.tile(np.array([temperature, top_k, top_p, 0.0, 0.0], np.float32), (rows, 1))


def _sampled_positions():
    at = np.arange(V)
    return (at % 1024) < 128


@pytest.mark.parametrize("mode", ["U", "G"])
def test_large_logits_where_the_sample_never_looks(sampler, device, mode):
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((4, V)).astype(np.float32)
    logits[:, ~_sampled_positions()] += 10.0  # the floor comes out far too low: the list overflows
    _check(sampler, device, _workload(logits, _options(4)), mode, expect_fallback=True)


@pytest.mark.parametrize("mode", ["U", "G"])
def test_large_logits_only_where_the_sample_looks(sampler, device, mode):
    rng = np.random.default_rng(2)
    logits = rng.standard_normal((4, V)).astype(np.float32)
    hot = np.flatnonzero(_sampled_positions())[::40]  # about 200 tokens, every one of them sampled
    logits[:, hot] += 12.0
    options = _options(4, top_k=250, top_p=1.0)  # more wanted than lie above the floor
    _check(sampler, device, _workload(logits, options), mode, expect_fallback=True)


def test_ordinary_rows_need_no_fallback(sampler, device):
    rng = np.random.default_rng(3)
    logits = (rng.standard_normal((8, V)) * 3).astype(np.float32)
    options = _options(8)
    options[3, 0] = 0.0  # a greedy row
    options[5, 1:4] = (0, 1.0, 0.05)  # a min-p row
    _check(sampler, device, _workload(logits, options), "U", expect_fallback=False)


@pytest.mark.parametrize("penalties", [(1.3, 0.0, 0.0), (1.0, 0.4, 0.0), (1.2, 0.3, 0.25), (0.8, 0.0, 0.0), (1.0, -0.5, 0.0), (1.0, 0.0, -0.3)])
def test_penalties_on_listed_rows(sampler, device, penalties):
    """Lowering penalties are applied to listed logits in place (bitmap, or counts when the
    frequency term is on); raising ones make the block fetch every history token."""
    rng = np.random.default_rng(4)
    rows = 6
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    history = rng.integers(0, V, (rows, 300)).astype(np.int32)
    top = np.argsort(-logits, axis=1)[:, :24]
    history[:, :24] = top  # the row's best tokens are history tokens, some of them twice
    history[:, 24:30] = top[:, :6]
    options = _options(rows, top_k=50, top_p=0.95)
    options[2, 0] = 0.0
    w = _workload(logits, options, history=history, penalties=np.tile(np.array(penalties, np.float32), (rows, 1)))
    _check(sampler, device, w, "U")
    _check(sampler, device, w, "G")


def test_rows_with_minus_infinity(sampler, device):
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal((4, V)) * 2).astype(np.float32)
    logits[0, rng.integers(0, V, 500)] = -np.inf
    logits[1, :] = -np.inf
    logits[1, 777] = 0.5  # one finite token: no floor can be guessed, the row is streamed
    logits[2, : V // 2] = -np.inf
    logits[3, ::3] = -np.inf
    _check(sampler, device, _workload(logits, _options(4)), "U")


def test_filter_path_off_gives_the_same_rows(sampler, device):
    from leat_b200 import workloads

    w = workloads.config2()
    on = helpers.gpu_run(sampler, w, "U", device, width=8)
    sampler.tune_filter(False)
    try:
        off = helpers.gpu_run(sampler, w, "U", device, width=8)
    finally:
        sampler.tune_filter(True)
    for name in ("ids", "greedy", "kept", "cut", "prob_ids", "probs"):
        np.testing.assert_array_equal(getattr(on, name).cpu().numpy(), getattr(off, name).cpu().numpy(), err_msg=name)


@pytest.mark.parametrize("mode", ["U", "G"])
def test_shards_whose_lists_fail_are_streamed_again(device, mode):
    """Vocabulary shards take the filter path too; a shard row whose list does not hold up is marked
    and streamed by a second launch, so the gathered candidates are complete either way."""
    from leat_b200 import workloads
    from tests.test_gpu_sharded_and_masks import _sharded_on_one_gpu

    rng = np.random.default_rng(9)
    rows, vocab, parts = 6, 4 * V, 4
    logits = rng.standard_normal((rows, vocab)).astype(np.float32)
    at = np.arange(vocab)
    # shard 0: large logits where its sample never looks; shard 1: only where it does; 2 and 3 plain
    logits[:, (at < V) & ((at % 1024) >= 128)] += 6.0
    hot = np.flatnonzero((at >= V) & (at < 2 * V) & ((at % 1024) < 128))[::50]
    logits[:, hot] += 9.0
    options = _options(rows, top_k=60, top_p=0.98)
    options[1, 0] = 0.0
    history = rng.integers(0, vocab, (rows, 128)).astype(np.int32)
    penalties = np.tile(np.array([1.2, 0.1, 0.0], np.float32), (rows, 1))
    w = workloads.Workload("case", logits, options, penalties, history, rng.random(rows, dtype=np.float32),
                           np.arange(rows, dtype=np.uint32) + 5, np.full(rows, 9, np.int32))  # fmt: skip
    got = _sharded_on_one_gpu(device, w, parts, mode)
    want = helpers.oracle_run(w, mode)
    helpers.compare(want, got, 64, max_fragile=1)
