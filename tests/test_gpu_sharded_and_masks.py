"""GPU parity of the vocabulary-sharded entry points (emulated on one GPU: the slices of N ranks
are selected one after the other, laid out as an all-gather would leave them, and finished once),
of the dense `seen` mask on the streaming path, and of the draft-verification kernel."""

import ctypes as C

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu


def _sharded_on_one_gpu(device, w, parts, mode, cap=128, k_max=64, width=64, dtype=None):
    import torch

    from leat_b200 import _lib, workloads
    from leat_b200.sampler import Sampled, Sampler, _stream

    t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
    rows, vocab = w.rows, w.vocab
    widest = max(b - a for a, b in (workloads.shard_bounds(vocab, parts, r) for r in range(parts)))
    sampler = Sampler(rows, max(widest, 8), k_max, device)
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    options, penalties, history, uniform, position = t(w.options), t(w.penalties), t(w.history), t(w.uniform), t(w.position)
    value = torch.zeros((parts, rows, cap), dtype=torch.float32, device=device)
    ids = torch.zeros((parts, rows, cap), dtype=torch.int32, device=device)
    count = torch.zeros((parts, rows), dtype=torch.int32, device=device)
    best = torch.zeros((parts, rows), dtype=torch.int64, device=device)
    for r in range(parts):
        start, stop = workloads.shard_bounds(vocab, parts, r)
        part = torch.as_tensor(np.ascontiguousarray(w.logits[:, start:stop])).to(device)
        part = part if dtype is None else part.to(dtype)  # (the slices' format on the device)
        a, keep = sampler._args(part, options, seed, position, None, history, None, penalties,
                                uniform if mode == "U" else None, 0, start, vocab)  # fmt: skip
        _lib.check(_lib.lib.leat_topk_local(sampler.handle, C.byref(a), value[r].data_ptr(), ids[r].data_ptr(),
                                            count[r].data_ptr(), best[r].data_ptr(), cap, _stream()), "leat_topk_local")  # fmt: skip
        torch.cuda.synchronize()
        assert int(count[r].min()) >= 0
    dummy = torch.empty((rows, 4), dtype=torch.float32, device=device)
    a, keep = sampler._args(dummy, options, seed, position, None, None, None, None, uniform if mode == "U" else None, 0)
    a.vocab, a.vocab_total = vocab, vocab
    out = Sampled(torch.empty((rows, 1), dtype=torch.int32, device=device),
                  status=torch.zeros(1, dtype=torch.int32, device=device))
    out.greedy = torch.empty(rows, dtype=torch.int32, device=device)
    out.cut = torch.empty(rows, dtype=torch.float32, device=device)
    out.kept = torch.empty(rows, dtype=torch.int32, device=device)
    out.probs = torch.empty((rows, width), dtype=torch.float32, device=device)
    out.prob_ids = torch.empty((rows, width), dtype=torch.int32, device=device)
    a.out_ids, a.status, a.out_greedy = out.ids.data_ptr(), out.status.data_ptr(), out.greedy.data_ptr()
    a.out_cut, a.out_kept = out.cut.data_ptr(), out.kept.data_ptr()
    a.out_probs, a.out_prob_ids, a.out_width = out.probs.data_ptr(), out.prob_ids.data_ptr(), width
    _lib.check(_lib.lib.leat_sample_from_candidates(sampler.handle, C.byref(a), value.data_ptr(), ids.data_ptr(),
                                                    count.data_ptr(), best.data_ptr(), parts, cap, _stream()),
               "leat_sample_from_candidates")  # fmt: skip
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("parts", [2, 4, 8])
@pytest.mark.parametrize("mode", ["U", "G"])
def test_sharded_equals_single_device_oracle(device, parts, mode):
    from leat_b200 import workloads

    w = workloads.config5(rows=24, vocab=201088)
    w.options[3, 0] = 0.0  # a greedy row among them
    got = _sharded_on_one_gpu(device, w, parts, mode)
    want = helpers.oracle_run(w, mode)
    helpers.compare(want, got, 64, max_fragile=1)


def test_dense_seen_mask_on_the_streaming_path(device):
    """leat's own form of the penalty input: a (B, V) bool mask, here on a vocabulary large enough
    to take the streaming path, with and without a history beside it."""
    import torch

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler
    from oracle import sampler_oracle as oracle

    w = workloads.config2(rows=6, vocab=151936)
    rng = np.random.default_rng(7)
    seen = np.zeros((w.rows, w.vocab), bool)
    for b in range(w.rows):
        seen[b, rng.integers(0, w.vocab, 700)] = True
        seen[b, np.argsort(-w.logits[b])[:5]] = True  # the likeliest tokens too
    w.options[:, 4] = 1.3  # presence penalty
    w.options[2, 0] = 0.0  # a greedy row
    sampler = Sampler(w.rows, w.vocab, 256, device)
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    for history in (None, w.history):
        penalties = None if history is None else w.penalties
        got = sampler.sample_full(t(w.logits), t(w.options), seed, t(w.position), t(seen),
                                  history=None if history is None else t(history),
                                  penalties=None if penalties is None else t(penalties),
                                  uniform=t(w.uniform), width=128, want_greedy=True, want_cut=True)  # fmt: skip
        want = oracle.sample(w.logits, w.options, w.seed, w.position, seen, history=history, penalties=penalties,
                             uniform_draws=w.uniform, order="block")  # fmt: skip
        helpers.compare(want, got, 128, max_fragile=0)


def test_verify_draft_accepts_and_rejects(device):
    import torch

    from leat_b200 import speculative
    from oracle import sampler_oracle as oracle

    rng = np.random.default_rng(3)
    sampled = rng.integers(0, 50, (16, 9)).astype(np.int32)
    drafted = sampled[:, :8].copy()
    for i in range(16):  # sequence i keeps i % 9 drafts
        if i % 9 < 8:
            drafted[i, i % 9] += 1
    greedy = sampled.copy()
    greedy[:, 5] += 1
    d, s, g = (torch.as_tensor(x).to(device) for x in (drafted, sampled, greedy))
    accepted, tokens = speculative.verify_draft(d, s)
    kept, toks = oracle.verify_draft(drafted, sampled)
    np.testing.assert_array_equal(accepted.cpu().numpy(), kept)
    np.testing.assert_array_equal(tokens.cpu().numpy(), toks)
    assert kept.tolist() == [i % 9 for i in range(16)]
    accepted, tokens = speculative.verify_draft(d, s, greedy=g)
    kept, toks = oracle.verify_draft_greedy(drafted, greedy, sampled)
    np.testing.assert_array_equal(accepted.cpu().numpy(), kept)
    np.testing.assert_array_equal(tokens.cpu().numpy(), toks)


def test_sharded_sampler_over_nccl_with_one_rank(device):
    """The host class end to end on a real process group with both exchanges (one rank: the
    all-gather of the packed records is then a copy, and the peer exchange stores into the rank's
    own region), against the oracle."""
    import os
    import socket

    import torch
    import torch.distributed as dist

    from leat_b200 import workloads
    from leat_b200.sharded import ShardedSampler

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    try:
        w = workloads.config5(rows=16, vocab=201088)
        t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
        seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
        want = helpers.oracle_run(w, "U")
        sharded = ShardedSampler(w.rows, w.vocab, k_max=64, cap=128, device=device, exchange="collective")
        got = sharded.sample(t(w.logits), t(w.options), seed, t(w.position), history=t(w.history),
                             penalties=t(w.penalties), uniform=t(w.uniform), width=64)  # fmt: skip
        torch.cuda.synchronize()
        helpers.compare(want, got, 64, max_fragile=0)
        peer = ShardedSampler(w.rows, w.vocab, k_max=64, cap=128, device=device, exchange="peer")
        assert peer.exchange_kind == "peer"
        for _ in range(3):
            got = peer.sample(t(w.logits), t(w.options), seed, t(w.position), history=t(w.history),
                              penalties=t(w.penalties), uniform=t(w.uniform))  # fmt: skip
            torch.cuda.synchronize()
            helpers.compare(want, got, 0, max_fragile=0)
            np.testing.assert_array_equal(got.kept.cpu().numpy(), want.kept)
            np.testing.assert_array_equal(got.cut.cpu().numpy(), want.cut)
        peer.close()
    finally:
        dist.destroy_process_group()


def test_sparse_slot_history_equals_the_dense_mask(device):
    """leat keeps a dense (slots, vocab) mask of generated tokens; SlotHistory keeps their ids.  A
    presence penalty through either gives the same tokens, cuts and survivors (the dense mask on
    the streaming kernel, the ids on the filter path)."""
    import torch

    from leat_b200.history import SlotHistory, dense_mask
    from leat_b200.sampler import Sampler

    rng = np.random.default_rng(31)
    slots, vocab, rows = 8, 50048, 5
    special = [5, 6, 7]
    h = SlotHistory(slots, 128, vocab, special_ids=special, device=device)
    for _ in range(60):
        which = torch.as_tensor(rng.permutation(slots)[:rows].copy())
        tokens = rng.integers(0, vocab, rows)
        tokens[rng.random(rows) < 0.1] = 6
        h.append(which, torch.as_tensor(tokens))
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    step_slots = torch.as_tensor([6, 1, 3, 0, 4])
    history, length = h.rows(step_slots)
    best = np.argsort(-logits, axis=1)[:, :5]
    history[:, :5] = torch.as_tensor(best.astype(np.int32)).to(device)  # make the penalty matter
    length = torch.clamp(length, min=5)
    seen = dense_mask(history, vocab, length)
    options = np.tile(np.array([0.8, 40, 0.95, 0.0, 1.5], np.float32), (rows, 1))
    options[2, 0] = 0.0
    sampler = Sampler(rows, vocab, 64, device)
    t = lambda x: torch.as_tensor(x).to(device)  # noqa: E731
    seed = torch.as_tensor(np.arange(rows, dtype=np.int64)).to(device).to(torch.uint32)
    position = t(np.full(rows, 7, np.int32))
    uniform = t(rng.random(rows, dtype=np.float32))
    penalties = t(np.tile(np.array([1.0, 1.5, 0.0], np.float32), (rows, 1)))
    sparse = sampler.sample_full(t(logits), t(options), seed, position, history=history, history_len=length,
                                 penalties=penalties, uniform=uniform, width=40, want_greedy=True, want_cut=True)  # fmt: skip
    dense = sampler.sample_full(t(logits), t(options), seed, position, seen.to(torch.uint8), uniform=uniform, width=40,
                                want_greedy=True, want_cut=True)  # fmt: skip
    torch.cuda.synchronize()
    # each against the CPU oracle given the same tokens (as ids and as the mask), then one against the other
    from oracle import sampler_oracle as oracle

    hist, lens = history.cpu().numpy(), length.cpu().numpy()
    want = oracle.sample(logits, options, np.arange(rows), 7, history=hist, history_len=lens,
                         penalties=np.tile(np.array([1.0, 1.5, 0.0], np.float32), (rows, 1)),
                         uniform_draws=uniform.cpu().numpy(), order="block")  # fmt: skip
    helpers.compare(want, sparse, 40, max_fragile=0)
    want_dense = oracle.sample(logits, options, np.arange(rows), 7, seen.cpu().numpy(), uniform_draws=uniform.cpu().numpy(), order="block")
    helpers.compare(want_dense, dense, 40, max_fragile=0)
    for name in ("ids", "greedy", "kept", "cut", "prob_ids", "probs"):
        a, b = getattr(sparse, name).cpu().numpy(), getattr(dense, name).cpu().numpy()
        if name == "cut":
            a, b = a[options[:, 0] > 0], b[options[:, 0] > 0]
        np.testing.assert_array_equal(a, b, err_msg=name)
