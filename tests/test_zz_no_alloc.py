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
    # and both against the CPU oracle, not only against each other
    want = helpers.oracle_run(w, mode)
    helpers.compare(want, static, width, max_fragile=1)
    helpers.compare(want, with_workspace, width, max_fragile=1)
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


def test_static_scratch_edges(device):
    """What the header promises beside the main path: rows with top_k above 64 are settled by the
    multi-pass routine (status bit FALLBACK) and still equal the oracle; 16-bit logits are refused;
    a call with no rows clears the status word on request and launches nothing."""
    import torch

    from leat_b200 import _lib, workloads
    from leat_b200.sampler import Sampler, sample_static
    from tests import helpers

    w = workloads.config2(rows=6, vocab=50048)
    w.options[:, 1] = 100.0  # top_k beyond the 64 the fixed scratch selects in one pass
    t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
    got = sample_static(t(w.logits), t(w.options), None, t(w.position), history=t(w.history), penalties=t(w.penalties),
                        uniform=t(w.uniform), width=128, want_greedy=True)  # fmt: skip
    torch.cuda.synchronize()
    assert int(got.status.item()) & _lib.STATUS_FALLBACK
    want = helpers.oracle_run(w, "U", order="sequential")
    firm = want.margin >= helpers.FRAGILE
    np.testing.assert_array_equal(got.ids.cpu().numpy().ravel()[firm], want.ids.ravel()[firm])
    np.testing.assert_array_equal(got.kept.cpu().numpy()[firm], want.kept[firm])
    np.testing.assert_array_equal(got.cut.cpu().numpy()[firm], want.cut[firm])
    with pytest.raises(ValueError):
        sample_static(t(w.logits).to(torch.bfloat16), t(w.options), uniform=t(w.uniform))
    args, keep = Sampler._args(None, torch.zeros((0, 1024), device=device), t(w.options[:1]), None, 0, None, None, None,
                               None, None, 0)  # fmt: skip
    status = torch.full((1,), 7, dtype=torch.int32, device=device)
    args.status, args.out_ids = status.data_ptr(), status.data_ptr()
    assert _lib.lib.leat_sample_static(C.byref(args), None) == _lib.OK
    torch.cuda.synchronize()
    assert int(status.item()) == 0
