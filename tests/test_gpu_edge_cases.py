"""Edges of the sampling path against the CPU oracle: no rows, one-token and unaligned
vocabularies, the vocabulary sizes around which the launch sequence changes, padded rows,
top_k at and beyond the vocabulary, a temperature below the clamp, min_p = 1, rows of equal
logits (every token ties), empty and partly filled histories, options given once for all rows,
and the full-size vocabulary-sharded configuration's rows by their invariants."""

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler(device):
    from leat_b200.sampler import Sampler

    return Sampler(512, 262144, 256, device)


def _workload(logits, options, history=None, penalties=None, seed=3):
    from leat_b200 import workloads

    rows = logits.shape[0]
    rng = np.random.default_rng(seed)
    return workloads.Workload("case", logits, options, penalties, history, rng.random(rows, dtype=np.float32),
                              np.arange(rows, dtype=np.uint32) + 17, np.full(rows, 2, np.int32))  # fmt: skip


def _options(rows, temperature=0.9, top_k=20, top_p=0.9, min_p=0.0):
    return np.tile(np.array([temperature, top_k, top_p, min_p, 0.0], np.float32), (rows, 1))


def test_no_rows(sampler, device):
    import torch

    logits = torch.empty((0, 4096), dtype=torch.float32, device=device)
    options = torch.empty((0, 5), dtype=torch.float32, device=device)
    seed = torch.empty(0, dtype=torch.uint32, device=device)
    position = torch.empty(0, dtype=torch.int32, device=device)
    got = sampler.sample_full(logits, options, seed, position)
    torch.cuda.synchronize()
    assert got.ids.shape[0] == 0 and sampler.last_launches == 0


@pytest.mark.parametrize("vocab", [1, 2, 5, 33, 4097, 16380, 16384, 16388, 16390, 40000])
@pytest.mark.parametrize("mode", ["U", "G"])
def test_vocabulary_sizes(sampler, device, vocab, mode):
    rng = np.random.default_rng(vocab)
    rows = 5
    logits = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    options = _options(rows)
    options[1, 0] = 0.0
    options[2, 1:3] = (0, 1.0)  # no cut at all
    options[3, 1] = vocab + 10  # top_k beyond the vocabulary
    options[4, 1] = vocab
    w = _workload(logits, options)
    # (no probabilities asked for: rows without a cut on a vocabulary beyond k_max are finished by an
    # argmax or by the multi-pass routine, which do not list them)
    got = helpers.gpu_run(sampler, w, mode, device, width=0)
    want = helpers.oracle_run(w, mode, order="sequential" if vocab > 256 else "block")
    helpers.compare(want, got, 0, max_fragile=1)
    import torch

    torch.cuda.synchronize()
    kept, cut = got.kept.cpu().numpy(), got.cut.cpu().numpy()
    for b in (0, 3, 4):
        if want.margin[b] >= helpers.FRAGILE:
            assert kept[b] == want.kept[b] and cut[b] == want.cut[b], (b, kept[b], want.kept[b], cut[b], want.cut[b])


@pytest.mark.parametrize("vocab, stride", [(32768, 32768 + 64), (1000, 1024), (20000, 20004)])
def test_padded_rows(sampler, device, vocab, stride):
    import torch

    rng = np.random.default_rng(stride)
    rows = 4
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    w = _workload(logits, _options(rows, top_k=30))
    padded = torch.full((rows, stride), 99.0, dtype=torch.float32, device=device)  # the padding would win if read
    padded[:, :vocab] = torch.as_tensor(logits).to(device)
    got = helpers.gpu_run(sampler, w, "U", device, width=32, logits=padded[:, :vocab])
    helpers.compare(helpers.oracle_run(w, "U"), got, 32, max_fragile=1)


def test_tiny_temperature_and_min_p_one(sampler, device):
    rng = np.random.default_rng(8)
    rows, vocab = 4, 50048
    logits = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    options = _options(rows)
    options[0, 0] = 1e-8  # clamped to 1e-6: a near-greedy draw
    options[1] = (1.0, 0, 1.0, 1.0, 0.0)  # min_p = 1: only the top score survives
    options[2] = (0.7, 0, 1.0, 0.999, 0.0)
    options[3] = (1.5, 1, 1.0, 0.0, 0.0)  # top_k = 1
    w = _workload(logits, options)
    for mode in ("U", "G"):
        got = helpers.gpu_run(sampler, w, mode, device, width=8)
        want = helpers.oracle_run(w, mode)
        helpers.compare(want, got, 8, max_fragile=1)
        assert got.kept.cpu().numpy()[1] == 1 and got.kept.cpu().numpy()[3] == 1


@pytest.mark.parametrize("vocab", [300, 20000])
def test_rows_of_equal_logits(sampler, device, vocab):
    """Every token ties at the k-th score, so every token survives and the draw is over all."""
    rows = 3
    logits = np.full((rows, vocab), 0.25, np.float32)
    logits[2, 7] = 1.0  # one better token, the rest tie
    options = _options(rows, top_k=10, top_p=1.0)
    w = _workload(logits, options)
    got = helpers.gpu_run(sampler, w, "U", device, width=0)
    want = helpers.oracle_run(w, "U", order="sequential")
    import torch

    torch.cuda.synchronize()
    assert int(got.status.item()) & 4 == 0
    np.testing.assert_array_equal(got.kept.cpu().numpy(), want.kept)
    np.testing.assert_array_equal(got.greedy.cpu().numpy(), want.greedy)
    ids = got.ids.cpu().numpy().ravel()
    for b in range(rows):
        assert ids[b] == want.ids[b, 0] or want.margin[b] < 1e-4


def test_histories_of_different_lengths(sampler, device):
    import torch

    rng = np.random.default_rng(12)
    rows, vocab, cap = 6, 50048, 64
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    lengths = np.array([0, 1, 17, 64, 0, 33], np.int32)
    history = rng.integers(0, vocab, (rows, cap)).astype(np.int32)
    best = np.argsort(-logits, axis=1)[:, :8]
    history[:, :8] = best
    penalties = np.tile(np.array([1.3, 0.5, 0.2], np.float32), (rows, 1))
    options = _options(rows, top_k=40, top_p=0.95)
    seed = np.arange(rows, dtype=np.uint32)
    position = np.full(rows, 4, np.int32)
    uniform = rng.random(rows, dtype=np.float32)
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    got = sampler.sample_full(t(logits), t(options), torch.as_tensor(seed.astype(np.int64)).to(device).to(torch.uint32),
                              t(position), history=t(history), history_len=t(lengths), penalties=t(penalties),
                              uniform=t(uniform), width=16, want_greedy=True, want_cut=True)  # fmt: skip
    from oracle import sampler_oracle as oracle

    for b in range(rows):
        h = history[b : b + 1, : lengths[b]] if lengths[b] else None
        want = oracle.sample(logits[b : b + 1], options[b : b + 1], seed[b : b + 1], position[b : b + 1], history=h,
                             penalties=penalties[b : b + 1] if h is not None else None,
                             uniform_draws=uniform[b : b + 1])  # fmt: skip
        torch.cuda.synchronize()
        if want.margin[0] >= helpers.FRAGILE:
            assert got.ids.cpu().numpy()[b, 0] == want.ids[0, 0], b
            assert got.kept.cpu().numpy()[b] == want.kept[0] and got.cut.cpu().numpy()[b] == want.cut[0], b
        assert got.greedy.cpu().numpy()[b] == want.greedy[0], b


def test_options_given_once_for_all_rows(sampler, device):
    import torch

    rng = np.random.default_rng(13)
    rows, vocab = 7, 32768
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    one = np.array([[0.8, 25, 0.9, 0.0, 0.0]], np.float32)
    w = _workload(logits, np.tile(one, (rows, 1)))
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    got = sampler.sample_full(t(logits), t(one), seed, t(w.position), uniform=t(w.uniform), width=32,
                              want_greedy=True, want_cut=True)  # fmt: skip
    helpers.compare(helpers.oracle_run(w, "U"), got, 32, max_fragile=1)


def test_full_size_config5_properties(sampler, device):
    """B = 512, V = 201088 on one device: determinism, survivors, probabilities, and a sample of
    rows against the oracle."""
    import torch

    from leat_b200 import workloads

    w = workloads.config5()
    logits = torch.as_tensor(w.logits).to(device)
    got = helpers.gpu_run(sampler, w, "U", device, width=64, logits=logits)
    again = helpers.gpu_run(sampler, w, "U", device, width=64, logits=logits)
    torch.cuda.synchronize()
    assert torch.equal(got.ids, again.ids) and torch.equal(got.probs, again.probs)
    assert int(got.status.item()) == 0  # no row needed the multi-pass routine
    ids, kept = got.ids.cpu().numpy().ravel(), got.kept.cpu().numpy()
    probs, prob_ids = got.probs.cpu().numpy(), got.prob_ids.cpu().numpy()
    for b in range(w.rows):
        assert 1 <= kept[b] <= 64 and ids[b] in prob_ids[b, : kept[b]]
        assert abs(probs[b].sum() - 1) < 1e-5 and (np.diff(probs[b, : kept[b]]) <= 0).all()
    rows = np.arange(0, w.rows, 32)
    want = helpers.oracle_run(w, "U", rows=rows)
    for i, b in enumerate(rows):
        assert got.greedy.cpu().numpy()[b] == want.greedy[i]
        if want.margin[i] >= helpers.FRAGILE:
            assert ids[b] == want.ids[i, 0] and kept[b] == want.kept[i]
            np.testing.assert_array_equal(prob_ids[b, : kept[b]], want.prob_ids[i])
            np.testing.assert_allclose(probs[b, : kept[b]], want.probs[i], rtol=helpers.PROB_RTOL)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("mode", ["U", "G"])
def test_sixteen_bit_logits(sampler, device, dtype, mode):
    """bfloat16 and float16 logits (an lm_head's own output) are read as they are; both convert to
    float32 exactly, so the oracle on the converted values is the answer.  Rows without a list (no
    cut at all, top-p over the whole vocabulary) go through the multi-pass routine."""
    import torch

    rng = np.random.default_rng(21)
    rows, vocab = 8, 65536
    raw = torch.as_tensor((rng.standard_normal((rows, vocab)) * 3).astype(np.float32))
    raw[:, :50] += 6.0
    narrow = raw.to(getattr(torch, dtype))
    logits = narrow.to(torch.float32).numpy()  # what the sampler must see
    options = _options(rows, top_k=50, top_p=0.9)
    options[1, 0] = 0.0
    options[2] = (0.8, 0, 0.9, 0.0, 0.0)  # top-p with no top-k: multi-pass
    options[3] = (1.0, 0, 1.0, 0.0, 0.0)  # no cut at all
    options[4] = (0.7, 0, 1.0, 0.05, 0.0)  # min-p only
    history = rng.integers(0, vocab, (rows, 96)).astype(np.int32)
    history[:, :6] = np.argsort(-logits, axis=1)[:, :6]
    penalties = np.tile(np.array([1.2, 0.3, 0.1], np.float32), (rows, 1))
    penalties[6] = (0.9, 0.0, 0.0)  # raises logits: history tokens are fetched one by one
    w = _workload(logits, options, history=history, penalties=penalties)
    got = helpers.gpu_run(sampler, w, mode, device, width=0, logits=narrow.to(device))
    want = helpers.oracle_run(w, mode, order="sequential")
    torch.cuda.synchronize()
    assert int(got.status.item()) & 4 == 0
    ids, kept, cut = got.ids.cpu().numpy().ravel(), got.kept.cpu().numpy(), got.cut.cpu().numpy()
    np.testing.assert_array_equal(got.greedy.cpu().numpy(), want.greedy)
    soft = 0
    for b in range(rows):
        greedy_row = not options[b, 0] > 0
        ok = ids[b] == want.ids[b, 0] and (greedy_row or (kept[b] == want.kept[b] and cut[b] == want.cut[b]))
        if not ok:
            assert want.margin[b] < 1e-4, (b, ids[b], want.ids[b, 0], kept[b], want.kept[b], cut[b], want.cut[b])
            soft += 1
    assert soft <= 1
