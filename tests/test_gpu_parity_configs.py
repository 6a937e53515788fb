"""Parity of the CUDA path with the CPU oracle on the benchmark configurations' shapes, value
distributions and options: reduced sizes in full against the oracle, and the full sizes on a
sample of rows plus size-independent properties."""

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler(device):
    from leat_b200.sampler import Sampler

    return Sampler(512, 262144, 256, device)


SMALL = [
    (1, dict(rows=4, vocab=128256)),
    (2, dict(rows=16, vocab=151936)),
    (3, dict(rows=32, vocab=262144)),
    (5, dict(rows=48, vocab=201088)),
    (1, dict(rows=7, vocab=33333)),   # a vocabulary that is not a multiple of 4: scalar loads
    (3, dict(rows=9, vocab=5000)),
]  # fmt: skip


@pytest.mark.parametrize("config, size", SMALL)
@pytest.mark.parametrize("mode", ["U", "G"])
def test_config_matches_oracle(sampler, device, config, size, mode):
    from leat_b200 import workloads

    w = workloads.CONFIGS[config](**size)
    width = 256
    got = helpers.gpu_run(sampler, w, mode, device, width=width)
    want = helpers.oracle_run(w, mode)
    helpers.compare(want, got, width, max_fragile=1)


@pytest.mark.parametrize("threads, slices", [(128, 1), (256, 3), (512, 0), (256, 64), (512, 2)])
def test_launch_shape_does_not_change_results(sampler, device, threads, slices):
    from leat_b200 import workloads

    w = workloads.config2(rows=8, vocab=151936)
    want = helpers.oracle_run(w, "U")
    sampler.tune(threads, slices)
    try:
        got = helpers.gpu_run(sampler, w, "U", device, width=128)
        helpers.compare(want, got, 128, max_fragile=0)
    finally:
        sampler.tune(0, 0)


def test_divide_flag(sampler, device):
    from leat_b200 import _lib, workloads

    w = workloads.config2(rows=8, vocab=50000)
    got = helpers.gpu_run(sampler, w, "U", device, width=128, flags=_lib.FLAG_DIVIDE)
    helpers.compare(helpers.oracle_run(w, "U", scale="divide"), got, 128, max_fragile=0)


def test_full_size_config3_properties(sampler, device):
    """B = 256, V = 262144: a sample of rows against the oracle, and on every row: greedy rows
    return the greedy id, sampled ids are survivors, probabilities sum to one, and the call is
    deterministic."""
    import torch

    from leat_b200 import workloads

    w = workloads.config3()
    logits = torch.as_tensor(w.logits).to(device)
    got = helpers.gpu_run(sampler, w, "U", device, width=256, logits=logits)
    again = helpers.gpu_run(sampler, w, "U", device, width=256, logits=logits)
    torch.cuda.synchronize()
    assert torch.equal(got.ids, again.ids) and torch.equal(got.probs, again.probs)
    ids, greedy, kept = got.ids.cpu().numpy().ravel(), got.greedy.cpu().numpy(), got.kept.cpu().numpy()
    probs, prob_ids = got.probs.cpu().numpy(), got.prob_ids.cpu().numpy()
    is_greedy = w.options[:, 0] == 0
    assert is_greedy.sum() == 64
    np.testing.assert_array_equal(ids[is_greedy], greedy[is_greedy])
    for b in np.nonzero(~is_greedy)[0]:
        assert 1 <= kept[b] <= 256 and ids[b] in prob_ids[b, : kept[b]]
        assert abs(probs[b].sum() - 1) < 1e-5 and (np.diff(probs[b, : kept[b]]) <= 0).all()
    rows = np.arange(0, 256, 16)
    want = helpers.oracle_run(w, "U", rows=rows)
    for i, b in enumerate(rows):
        assert greedy[b] == want.greedy[i]
        if want.margin[i] >= helpers.FRAGILE:
            assert ids[b] == want.ids[i, 0]
            if not is_greedy[b]:
                assert kept[b] == want.kept[i]
                np.testing.assert_array_equal(prob_ids[b, : kept[b]], want.prob_ids[i])
                np.testing.assert_allclose(probs[b, : kept[b]], want.probs[i], rtol=helpers.PROB_RTOL)


def test_config4_draft_verification(sampler, device):
    import torch

    from leat_b200 import speculative, workloads
    from oracle import sampler_oracle as oracle

    w = workloads.config4()
    n, drafts = w.meta["sequences"], w.meta["drafts"]
    got = helpers.gpu_run(sampler, w, "U", device, width=64)
    want = helpers.oracle_run(w, "U")
    helpers.compare(want, got, 64, max_fragile=0)
    drafted = torch.as_tensor(w.drafted).to(device)
    sampled = got.ids.reshape(n, drafts + 1)
    accepted, tokens = speculative.verify_draft(drafted, sampled)
    kept, toks = oracle.verify_draft(w.drafted, want.ids.reshape(n, drafts + 1))
    np.testing.assert_array_equal(accepted.cpu().numpy(), kept)
    np.testing.assert_array_equal(tokens.cpu().numpy(), toks)
    accepted, tokens = speculative.verify_draft(drafted, sampled, greedy=got.greedy.reshape(n, drafts + 1))
    kept, toks = oracle.verify_draft_greedy(w.drafted, want.greedy.reshape(n, drafts + 1),
                                            want.ids.reshape(n, drafts + 1))  # fmt: skip
    np.testing.assert_array_equal(accepted.cpu().numpy(), kept)
    np.testing.assert_array_equal(tokens.cpu().numpy(), toks)
