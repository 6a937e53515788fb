"""The sparse per-slot history that replaces leat's dense (slots, vocab) mask (leat/engine.py:167-173,
768-781, 664-675), on CPU tensors: what it records equals what the dense mask would hold."""

import numpy as np
import torch

from leat_b200.history import SlotHistory, dense_mask, options_row


def _dense_reference(vocab, special, events):
    """leat's bookkeeping, step by step: a (slots, vocab) boolean array."""
    slots = 1 + max(s for kind, payload in events for s in (payload[0] if kind == "append" else payload))
    seen = np.zeros((slots, vocab), bool)
    for kind, payload in events:
        if kind == "reset":
            for s in payload:
                seen[s] = False
        else:
            for s, t in zip(*payload):
                if t not in special:
                    seen[s, t] = True
    return seen


def test_appends_and_resets_match_the_dense_mask():
    rng = np.random.default_rng(0)
    vocab, slots, special = 500, 6, {3, 7, 499}
    h = SlotHistory(slots, 64, vocab, special_ids=special)
    events = []
    for step in range(40):
        if step % 11 == 5:
            which = [int(rng.integers(slots))]
            h.reset(torch.tensor(which))
            events.append(("reset", which))
        rows = rng.permutation(slots)[: rng.integers(1, slots + 1)]
        tokens = rng.integers(0, vocab, len(rows))
        tokens[rng.random(len(rows)) < 0.2] = 7  # markup is never recorded
        h.append(torch.tensor(rows), torch.tensor(tokens))
        events.append(("append", (rows.tolist(), tokens.tolist())))
    want = _dense_reference(vocab, special, events)
    got = h.dense(torch.arange(slots)).numpy()
    np.testing.assert_array_equal(got, want[:slots])
    ids, length = h.rows(torch.arange(slots))
    assert ids.dtype == torch.int32 and length.dtype == torch.int32 and int(length.max()) <= 64


def test_a_full_slot_overwrites_its_oldest_tokens():
    h = SlotHistory(2, 4, 100)
    for t in range(10):
        h.append(torch.tensor([1]), torch.tensor([t]))
    ids, length = h.rows(torch.tensor([1, 0]))
    assert sorted(ids[0].tolist()) == [6, 7, 8, 9] and int(length[0]) == 4
    assert ids[1].tolist() == [-1, -1, -1, -1] and int(length[1]) == 0


def test_rows_of_a_speculative_run():
    vocab = 50
    h = SlotHistory(3, 8, vocab, special_ids=[9])
    h.append(torch.tensor([0, 2]), torch.tensor([11, 12]))
    run = torch.tensor([[20, 9, 21], [30, 31, 32]])  # two sequences (slots 2 and 0), three tokens each
    rows = h.rows_of_run(torch.tensor([2, 0]), run)
    assert rows.shape == (6, 8 + 3)
    seen = dense_mask(rows, vocab).numpy()
    expect = [{12, 20}, {12, 20}, {12, 20, 21}, {11, 30}, {11, 30, 31}, {11, 30, 31, 32}]  # 9 is markup
    for r, want in enumerate(expect):
        assert set(np.nonzero(seen[r])[0].tolist()) == want, r


def test_request_to_option_rows():
    from leat_b200.sampler import Sampling

    options, penalties = options_row(Sampling(0.7, 40, 0.9, 0.05, 0.5), frequency_penalty=0.2, repetition_penalty=1.1)
    assert options == [0.7, 40.0, 0.9, 0.05, 0.5] and penalties == [1.1, 0.5, 0.2]


def test_request_mapping_follows_the_reference_server():
    """leat's own mapping cases (tests/test_server.py:255-266 of the reference): OpenAI's fields and
    vLLM's, top_k of -1 keeping every token as 0; absent or null fields take OpenAI's defaults."""
    import pytest

    from leat_b200.history import sampling_from_request
    from leat_b200.sampler import Sampling

    body = {"temperature": 0.5, "top_k": -1, "top_p": 0.9, "min_p": 0.05, "presence_penalty": 1.5, "max_tokens": 9, "seed": 3}
    sampling, frequency, repetition = sampling_from_request(body)
    assert sampling == Sampling(0.5, 0, 0.9, 0.05, 1.5) and (frequency, repetition) == (0.0, 1.0)
    sampling, _, _ = sampling_from_request({"stop": ["", "y"], "top_p": None})
    assert sampling == Sampling(1.0)
    # a model's own defaults, which a request's fields override (leat/defaults.py)
    sampling, _, _ = sampling_from_request({"top_k": 20}, defaults={"temperature": 0.6, "top_k": 40, "top_p": 0.95})
    assert sampling == Sampling(0.6, 20, 0.95)
    # the ranges of leat/server.py:84-109 and leat/defaults.py:26-29
    for bad in ({"temperature": 2.5}, {"temperature": -0.1}, {"top_p": 1.2}, {"min_p": -0.5}, {"presence_penalty": 3},
                {"top_k": 1.5}, {"top_k": (1 << 20) + 1}, {"temperature": "hot"}, {"top_p": True},
                {"frequency_penalty": 2.5}, {"repetition_penalty": 0}, {"repetition_penalty": 2.5}):  # fmt: skip
        with pytest.raises(ValueError):
            sampling_from_request(bad)
    # the two penalties leat's server refuses are taken here
    _, frequency, repetition = sampling_from_request({"frequency_penalty": 0.4, "repetition_penalty": 1.2})
    assert (frequency, repetition) == (0.4, 1.2)
    with pytest.raises(ValueError):
        options_row(Sampling(3.0))
