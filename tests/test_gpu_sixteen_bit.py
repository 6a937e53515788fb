"""bfloat16 and float16 logits off the filter path: rows too narrow or too oddly sized for a list, a
dense `seen` mask, and vocabulary shards over both exchanges.  Both formats convert to float32
exactly, so the CPU oracle on the converted values is the answer, by the same parity rules."""

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu

FORMATS = ["bfloat16", "float16"]


def _rounded(logits, dtype):
    """The float32 values a 16-bit copy of `logits` holds."""
    import torch

    return torch.as_tensor(logits).to(getattr(torch, dtype)).to(torch.float32).numpy()


def _case(rows, vocab, dtype, seed):
    from leat_b200 import workloads

    rng = np.random.default_rng(seed)
    logits = _rounded((rng.standard_normal((rows, vocab)) * 3).astype(np.float32), dtype)
    options = np.tile(np.array([0.9, 20, 0.9, 0.0, 0.0], np.float32), (rows, 1))
    options[1, 0] = 0.0  # greedy
    options[2] = (0.7, 0, 1.0, 0.05, 0.0)  # min-p alone
    options[3, 1] = min(vocab, 64)
    history = rng.integers(0, vocab, (rows, 48)).astype(np.int32)
    top = np.argsort(-logits, axis=1)[:, :4]
    history[:, : top.shape[1]] = top
    penalties = np.tile(np.array([1.2, 0.3, 0.1], np.float32), (rows, 1))
    penalties[4] = (0.9, 0.0, 0.0)  # raises logits
    return workloads.Workload("case", logits, options, penalties, history, rng.random(rows, dtype=np.float32),
                              np.arange(rows, dtype=np.uint32) + 5, np.full(rows, 3, np.int32))  # fmt: skip


@pytest.mark.parametrize("dtype", FORMATS)
@pytest.mark.parametrize("vocab", [1, 7, 1000, 4099, 16392, 40001])
@pytest.mark.parametrize("mode", ["U", "G"])
def test_rows_without_a_list(device, dtype, vocab, mode):
    """Narrow rows and vocabularies that are not whole 16-byte vectors are streamed with plain loads."""
    import torch

    from leat_b200.sampler import Sampler

    w = _case(6, vocab, dtype, vocab)
    sampler = Sampler(8, 65536, 64, device)
    narrow = torch.as_tensor(w.logits).to(getattr(torch, dtype)).to(device)
    got = helpers.gpu_run(sampler, w, mode, device, width=64, logits=narrow)
    want = helpers.oracle_run(w, mode)
    helpers.compare(want, got, 64, max_fragile=1)


@pytest.mark.parametrize("dtype", FORMATS)
def test_dense_seen_mask(device, dtype):
    import torch

    from leat_b200.sampler import Sampler
    from oracle import sampler_oracle as oracle

    rows, vocab = 6, 65536
    w = _case(rows, vocab, dtype, 11)
    rng = np.random.default_rng(12)
    seen = np.zeros((rows, vocab), bool)
    for b in range(rows):
        seen[b, rng.integers(0, vocab, 500)] = True
        seen[b, np.argsort(-w.logits[b])[:5]] = True
    w.options[:, 4] = 1.1  # presence penalty
    sampler = Sampler(rows, vocab, 64, device)
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    got = sampler.sample_full(t(w.logits).to(getattr(torch, dtype)), t(w.options), seed, t(w.position), t(seen),
                              uniform=t(w.uniform), width=64, want_greedy=True, want_cut=True)  # fmt: skip
    want = oracle.sample(w.logits, w.options, w.seed, w.position, seen, uniform_draws=w.uniform, order="block")
    helpers.compare(want, got, 64, max_fragile=0)


@pytest.mark.parametrize("dtype", FORMATS)
@pytest.mark.parametrize("parts", [2, 8])
def test_shards_over_one_all_gather(device, dtype, parts):
    import torch

    from leat_b200 import workloads
    from tests.test_gpu_sharded_and_masks import _sharded_on_one_gpu

    w = workloads.config5(rows=16, vocab=201088)
    w.logits = _rounded(w.logits, dtype)
    w.options[3, 0] = 0.0
    got = _sharded_on_one_gpu(device, w, parts, "U", dtype=getattr(torch, dtype))
    helpers.compare(helpers.oracle_run(w, "U"), got, 64, max_fragile=1)


@pytest.mark.parametrize("dtype", FORMATS)
@pytest.mark.parametrize("vocab,parts", [(201088, 2), (201088, 8), (50048, 4)])
def test_shards_over_peer_memory(device, dtype, vocab, parts):
    """Listed slices (the filter reads the 16-bit logits) and slices too narrow for a list (streamed)."""
    import torch

    from leat_b200 import workloads
    from tests.test_gpu_peer_shards import PeerShardsOnOneGpu

    w = workloads.config5(rows=16, vocab=vocab)
    w.logits = _rounded(w.logits, dtype)
    w.options[3, 0] = 0.0
    w.options[5, 1:4] = (0.0, 1.0, 0.02)  # min-p alone
    emu = PeerShardsOnOneGpu(device, w.rows, w.vocab, parts)
    try:
        for mode in ("U", "G"):
            want = helpers.oracle_run(w, mode)
            for r, got in emu.step(w, mode, dtype=getattr(torch, dtype)).items():
                assert int(got.status.item()) & 12 == 0, f"rank {r}: status {int(got.status.item())}"
                helpers.compare(want, got, 0, max_fragile=1)
    finally:
        emu.close()
