"""GPU tests of what goes beyond leat's own call: the model's soft cap applied inside the sampler,
logits and options handed over as another framework's device buffers, an int position passed by
value, the device-side settle of a speculative step, and the limits on the history's length."""

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu


def _gpu(sampler, w, mode, device, **more):
    import torch

    t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    return sampler.sample_full(t(w.logits), t(w.options), seed, t(w.position), history=t(w.history), penalties=t(w.penalties),
                               uniform=t(w.uniform) if mode == "U" else None, want_greedy=True, want_cut=True, **more)  # fmt: skip


@pytest.mark.parametrize("mode", ["U", "G"])
@pytest.mark.parametrize("vocab", [151936, 5000])
def test_soft_cap_matches_the_oracle(device, mode, vocab):
    """tanh(logits / cap) * cap (leat/model.py:419-423) inside the sampler: on the list path (large
    vocabulary) and through the multi-pass routine (small one).  Ids, survivor sets and cuts are
    bit-exact, probabilities within 1e-6 relative: both sides evaluate the cap in double precision."""
    from leat_b200 import workloads
    from leat_b200.sampler import Sampler
    from oracle import sampler_oracle as oracle

    w = workloads.config2(rows=12, vocab=vocab)
    w.logits *= 4.0  # so that the cap bites: logits up to +-48 against a cap of 30
    w.options[3, 0] = 0.0  # a greedy row
    w.options[5, 1:4] = (40.0, 0.9, 0.0)  # top-k with top-p
    sampler = Sampler(w.rows, w.vocab, 256, device)
    got = _gpu(sampler, w, mode, device, width=128, softcap=30.0)
    want = oracle.sample(w.logits, w.options, w.seed, w.position, history=w.history, penalties=w.penalties,
                         uniform_draws=w.uniform if mode == "U" else None, order="block", softcap=30.0)  # fmt: skip
    # (the multi-pass routine sums in its own order: compare it in the plain order, ties exempted)
    if vocab < 16384:
        want = oracle.sample(w.logits, w.options, w.seed, w.position, history=w.history, penalties=w.penalties,
                             uniform_draws=w.uniform if mode == "U" else None, order="sequential", softcap=30.0)  # fmt: skip
        np.testing.assert_array_equal(got.greedy.cpu().numpy(), want.greedy)
        firm = want.margin >= helpers.FRAGILE
        np.testing.assert_array_equal(got.ids.cpu().numpy().ravel()[firm], want.ids.ravel()[firm])
        sampled = firm & (w.options[:, 0] > 0)
        np.testing.assert_array_equal(got.kept.cpu().numpy()[sampled], want.kept[sampled])
        np.testing.assert_array_equal(got.cut.cpu().numpy()[sampled], want.cut[sampled])
    else:
        helpers.compare(want, got, 128, max_fragile=1)
    # and the cap changes something: without it the greedy row's logit differs
    plain = oracle.sample(w.logits, w.options, w.seed, w.position, history=w.history, penalties=w.penalties,
                          uniform_draws=w.uniform if mode == "U" else None, order="block")  # fmt: skip
    assert not np.array_equal(plain.cut, want.cut)


class _Foreign:
    """A device buffer of "another framework": only the CUDA array interface, nothing of torch."""

    def __init__(self, tensor):
        self._keep = tensor
        self.__cuda_array_interface__ = tensor.__cuda_array_interface__


class _ForeignDlpack:
    def __init__(self, tensor):
        self._t = tensor

    def __dlpack__(self, stream=None):
        return self._t.__dlpack__(stream=stream)

    def __dlpack_device__(self):
        return self._t.__dlpack_device__()


def test_foreign_device_buffers_and_an_int_position(device):
    """leat's sample() takes its own framework's tensors and `position` as an int (leat/sampler.py:31-45):
    here logits, options and seed arrive through the CUDA array interface and DLPack (numba's device
    arrays when numba is there, else plain wrappers that expose nothing else), the position by value."""
    import torch

    import leat_b200
    from leat_b200 import workloads
    from oracle import sampler_oracle as oracle

    w = workloads.config1(rows=6, vocab=128256)
    w.position[:] = 37
    w.seed &= np.uint32(0x7FFFFFFF)  # (handed over as int32 words below)
    want = oracle.sample(w.logits, w.options, w.seed, 37, order="block")  # leat's own call: no history, hashed draw
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(w.seed.astype(np.int32)).to(device)
    kinds = [lambda x: _Foreign(x), lambda x: _ForeignDlpack(x)]
    try:
        from numba import cuda as numba_cuda

        kinds.append(lambda x: numba_cuda.as_cuda_array(x))
    except Exception:  # numba absent or without a driver binding: the wrappers above stand in
        pass
    for wrap in kinds:
        ids = leat_b200.sample(wrap(t(w.logits)), wrap(t(w.options)), wrap(seed), 37)
        torch.cuda.synchronize()
        assert isinstance(ids, torch.Tensor) and tuple(ids.shape) == (w.rows, 1)
        firm = want.margin >= helpers.FRAGILE
        np.testing.assert_array_equal(ids.cpu().numpy().ravel()[firm], want.ids.ravel()[firm])
        assert hasattr(ids, "__dlpack__") and hasattr(ids, "__cuda_array_interface__")  # goes back the same way


def test_settle_draft_on_the_device(device):
    """The history after a speculative step, and the next step's tokens, against the host loop
    (leat/engine.py:609-631, :677-686 restated in the oracle)."""
    import torch

    from leat_b200 import speculative
    from leat_b200.history import SlotHistory
    from oracle import sampler_oracle as oracle

    rng = np.random.default_rng(11)
    slots_total, capacity, vocab, n, drafts = 8, 16, 1000, 5, 3
    special = [5, 6, 7]
    h = SlotHistory(slots_total, capacity, vocab, special_ids=special, device=device)
    for _ in range(20):  # some tokens already there, rings partly wrapped
        which = torch.as_tensor(rng.permutation(slots_total)[:n].copy())
        h.append(which, torch.as_tensor(rng.integers(0, vocab, n)))
    ids0, count0 = h.ids.cpu().numpy().copy(), h.count.cpu().numpy().copy()
    text = np.ones(vocab, bool)
    text[special] = False
    slots = rng.permutation(slots_total)[:n].astype(np.int32)
    last = rng.integers(0, vocab, n).astype(np.int32)
    last[1] = 6  # markup: not recorded
    drafted = rng.integers(0, vocab, (n, drafts)).astype(np.int32)
    sampled = rng.integers(0, vocab, (n, drafts + 1)).astype(np.int32)
    accepted = np.array([0, 3, 1, 2, 3], np.int32)
    want_next, want_row = oracle.settle_draft(ids0, count0, capacity, text, slots, last, drafted, sampled, accepted)
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    nxt, row = speculative.settle_draft(h, t(slots), t(last), t(drafted), t(sampled), t(accepted))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(nxt.cpu().numpy(), want_next)
    np.testing.assert_array_equal(row.cpu().numpy(), want_row)
    np.testing.assert_array_equal(h.ids.cpu().numpy(), ids0)
    np.testing.assert_array_equal(h.count.cpu().numpy(), count0)


def test_history_length_limits(device):
    """A history of 4096 tokens per row is sampled (against the oracle); one the kernels' shared
    memory cannot hold is refused on the host, before anything is launched."""
    import torch

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler

    w = workloads.config5(rows=4, vocab=50048)
    rng = np.random.default_rng(2)
    w.history = rng.integers(0, w.vocab, (w.rows, 4096)).astype(np.int32)
    sampler = Sampler(w.rows, w.vocab, 256, device)
    got = helpers.gpu_run(sampler, w, "U", device, width=64)
    helpers.compare(helpers.oracle_run(w, "U"), got, 64, max_fragile=0)
    small = workloads.config5(rows=4, vocab=5000)  # the streaming kernel, which keeps the history in a hash table
    small.history = rng.integers(0, small.vocab, (small.rows, 4097)).astype(np.int32)
    with pytest.raises(ValueError, match="capacity"):
        helpers.gpu_run(sampler, small, "U", device, width=64)
    small.history = small.history[:, :4096].copy()
    got = helpers.gpu_run(sampler, small, "U", device, width=64)
    helpers.compare(helpers.oracle_run(small, "U"), got, 64, max_fragile=0)
    assert float(torch.ones(2, device=device).sum().item()) == 2.0
