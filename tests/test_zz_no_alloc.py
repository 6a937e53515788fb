"""The allocation-free entry point, leat_sample_static: for callers that cannot allocate device
memory where they sample (a server whose pool is fully committed, a binding that only receives
pointers), the library keeps the scratch of a call in a fixed array of its own.  Its results must
equal those of leat_sample with a caller-owned workspace, call after call: the array keeps what the
previous call left in it.  Collected last on purpose (zz), and written to pass alone in a fresh
process as well as after every other test."""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _both(device, w, mode, width):
    import torch

    from leat_b200 import _lib
    from leat_b200.sampler import Sampler, sample_static
    from tests import helpers

    sampler = Sampler(w.rows, w.vocab, 64, device)
    with_workspace = helpers.gpu_run(sampler, w, mode, device, width=width)
    t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    static = sample_static(t(w.logits), t(w.options), seed, t(w.position), history=t(w.history),
                           penalties=t(w.penalties), uniform=t(w.uniform) if mode == "U" else None,
                           width=width, want_greedy=True)  # fmt: skip
    torch.cuda.synchronize()
    assert int(static.status.item()) & _lib.STATUS_INTERNAL == 0
    return with_workspace, static


def _same(a, b):
    import torch

    assert torch.equal(a.ids, b.ids)
    assert torch.equal(a.greedy, b.greedy)
    assert torch.equal(a.kept, b.kept)
    assert torch.equal(a.prob_ids, b.prob_ids)
    np.testing.assert_allclose(b.probs.cpu().numpy(), a.probs.cpu().numpy(), rtol=1e-6, atol=0)
    np.testing.assert_array_equal(b.cut.cpu().numpy(), a.cut.cpu().numpy())


def test_static_scratch_matches_workspace_twice_in_a_row(device):
    from leat_b200 import workloads

    # two different calls back to back: the second starts from the first one's leftovers
    first = workloads.config2(rows=16, vocab=151936)
    second = workloads.config1(rows=5, vocab=128256)
    _same(*_both(device, first, "U", 64))
    _same(*_both(device, second, "G", 64))
    _same(*_both(device, first, "G", 64))


def test_static_scratch_rejects_what_it_cannot_hold(device):
    import torch

    from leat_b200 import _lib
    from leat_b200.sampler import sample_static

    options = torch.tensor([[1.0, 8, 1.0, 0.0, 0.0]], device=device)
    too_many = torch.zeros((65, 1024), device=device)
    too_wide = torch.zeros((1, (1 << 18) + 4), device=device)
    for logits in (too_many, too_wide):
        with pytest.raises(ValueError, match="capacity"):
            sample_static(logits, options, uniform=torch.zeros(logits.shape[0], device=device))
    args = _lib.SampleArgs()
    assert _lib.lib.leat_sample_static(C.byref(args), None) == _lib.E_ARGUMENT
