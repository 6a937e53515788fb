"""Rows the single pass cannot take go through the exact multi-pass kernel: top-p with no top-k on
a full vocabulary (leat's Llama default), top-k beyond the candidate buffer, massive ties at the
k-th score, and the supplied-uniform draw with no cut.  Checked against the CPU oracle; the cut
kernel also against the reference's own cases (leat tests/test_kernels.py:939-955), exactly rather
than within its histogram tolerance."""

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler(device):
    from leat_b200.sampler import Sampler

    return Sampler(64, 262144, 256, device)


def _run(sampler, device, logits, options, mode, seed=None, position=None, uniform=None, history=None, penalties=None):
    import torch

    from leat_b200 import workloads

    rows = logits.shape[0]
    w = workloads.Workload("case", logits, options, penalties, history,
                           uniform if uniform is not None else np.zeros(rows, np.float32),
                           seed if seed is not None else np.arange(rows, dtype=np.uint32),
                           position if position is not None else np.full(rows, 5, np.int32))  # fmt: skip
    got = helpers.gpu_run(sampler, w, mode, device, width=0)
    want = helpers.oracle_run(w, mode, order="sequential")
    torch.cuda.synchronize()
    return w, got, want


def _check(got, want, max_fragile=1):
    ids, kept, cut = got.ids.cpu().numpy().ravel(), got.kept.cpu().numpy(), got.cut.cpu().numpy()
    assert int(got.status.item()) & 4 == 0
    np.testing.assert_array_equal(got.greedy.cpu().numpy(), want.greedy)
    soft = 0
    for b in range(len(ids)):
        ok = ids[b] == want.ids[b, 0] and kept[b] == want.kept[b] and cut[b] == want.cut[b]
        if not ok:
            assert want.margin[b] < 1e-4, (b, ids[b], want.ids[b, 0], kept[b], want.kept[b], cut[b], want.cut[b], want.margin[b])
            soft += 1
    assert soft <= max_fragile


@pytest.mark.parametrize("mode", ["U", "G"])
def test_top_p_without_top_k_on_a_full_vocabulary(sampler, device, mode):
    rng = np.random.default_rng(11)
    logits = (rng.standard_normal((6, 128256)) * 3).astype(np.float32)
    logits[:, :40] += 9  # a head of likely tokens, as a model's logits have
    options = np.tile(np.array([0.6, 0, 0.9, 0.0, 0.0], np.float32), (6, 1))
    options[1, 2], options[2, 3], options[3, 2] = 0.5, 0.01, 0.0
    history = rng.integers(0, 128256, (6, 256)).astype(np.int32)
    penalties = np.tile(np.array([1.1, 0.2, 0.1], np.float32), (6, 1))
    _, got, want = _run(sampler, device, logits, options, mode, uniform=rng.random(6, dtype=np.float32),
                        history=history, penalties=penalties)  # fmt: skip
    assert int(got.status.item()) & 1  # the multi-pass kernel ran
    _check(got, want)


@pytest.mark.parametrize("mode", ["U", "G"])
def test_top_k_beyond_the_buffer_and_uniform_without_a_cut(sampler, device, mode):
    rng = np.random.default_rng(12)
    logits = (rng.standard_normal((4, 50000)) * 2.5).astype(np.float32)
    options = np.array([[1.0, 2000, 1.0, 0, 0], [0.8, 3000, 0.7, 0, 0], [1.0, 0, 1.0, 0, 0], [1.3, 600, 1.0, 0.001, 0]], np.float32)
    _, got, want = _run(sampler, device, logits, options, mode, uniform=rng.random(4, dtype=np.float32))
    _check(got, want)


@pytest.mark.parametrize("mode", ["U", "G"])
def test_ties_at_the_kth_score_all_survive(sampler, device, mode):
    rng = np.random.default_rng(13)
    flat = np.zeros((3, 40000), np.float32)
    flat[1, ::3] = 1.0  # a third of the row tied at the top
    flat[2] = np.round(rng.standard_normal(40000) * 2).astype(np.float32)  # few distinct values
    options = np.array([[1.0, 10, 1.0, 0, 0], [0.9, 50, 0.9, 0, 0], [1.0, 64, 0.95, 0, 0]], np.float32)
    _, got, want = _run(sampler, device, flat, options, mode, uniform=np.array([0.37, 0.81, 0.05], np.float32))
    assert got.kept.cpu().numpy().tolist() == want.kept.tolist()
    _check(got, want, max_fragile=0)


@pytest.mark.parametrize("rows, n", [(1, 248320), (5, 32000), (2, 300)])
def test_cutoff_cases_of_the_reference(device, rows, n):
    import torch

    from leat_b200 import ops
    from oracle import sampler_oracle as oracle

    rng = np.random.default_rng(n)
    x = (rng.standard_normal((rows, n)) * 2.5).astype(np.float32)
    x[:, : n // 100] += 9  # a head of likely tokens
    top_k = np.array([20, 0, 5, 1, 0][:rows], np.float32)
    top_p = np.array([0.95, 0.9, 1.0, 0.5, 0.0][:rows], np.float32)
    got = ops.cutoff(torch.as_tensor(x).to(device), torch.as_tensor(top_k).reshape(-1, 1),
                     torch.as_tensor(top_p).reshape(-1, 1), torch.zeros(rows, 1)).cpu().numpy()  # fmt: skip
    assert got.shape == (rows, 1)
    for b in range(rows):
        ranked = -np.sort(-x[b])
        c = oracle.cutoff_row(ranked, top_k[b], top_p[b], 0.0)
        top, by_k, by_p = oracle.cuts_f64(x[b], top_k[b], top_p[b])
        exact = np.float32(by_p if top_p[b] < 1 else by_k)
        if not (top_k[b] > 0 or top_p[b] < 1):
            exact = np.float32(-np.inf)
        assert got[b, 0] == c.cut or got[b, 0] == exact or c.margin < 1e-4, (b, got[b, 0], c.cut, exact)
