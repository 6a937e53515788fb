"""Pins the CPU oracle to the known answers the reference's own tests hold for the sampling path
(tests/test_sampler.py:37-93, tests/test_kernels.py:927-955, tests/helpers.py:354-361 of leat).
Runs without a GPU."""

import numpy as np
import pytest

from oracle import sampler_oracle as oracle

LOGITS = [2.0, 1.0, 0.0, -1.0, 0.5]


def values(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, presence_penalty=0.0):
    return [temperature, top_k, top_p, min_p, presence_penalty]


def draws(logits, sampling, seed, position, seen=None, **kw):
    options = np.array(sampling if isinstance(sampling[0], list) else [sampling], np.float32)
    seeds = np.array(seed if isinstance(seed, list) else [seed], np.uint32)
    return oracle.sample(np.array(logits, np.float32), options, seeds, position, seen, **kw).ids.ravel().tolist()


def frequencies(sampling, n=20000, rows=1000, **kw):
    got = [t for i in range(0, n, rows) for t in draws([LOGITS] * rows, sampling, list(range(i, i + rows)), 0, **kw)]
    return np.bincount(got, minlength=len(LOGITS)) / n


def softmax(logits, temperature=1.0):
    p = np.exp(np.array(logits) / temperature)
    return p / p.sum()


def test_greedy():
    assert draws([LOGITS, LOGITS[::-1]], values(), 0, 0) == [0, 4]


@pytest.mark.parametrize("order", ["sequential", "block"])
def test_temperature_matches_softmax(order):
    np.testing.assert_allclose(frequencies(values(0.7), order=order), softmax(LOGITS, 0.7), atol=0.015)


@pytest.mark.parametrize("sampling, kept", [
    (values(1.0, top_k=2), [0, 1]),
    (values(1.0, top_k=4, top_p=0.8), [0, 1, 4]),
    (values(1.0, top_p=0.5), [0]),
    (values(1.0, min_p=0.2), [0, 1, 4]),
])  # fmt: skip
def test_cut_tokens_never_drawn(sampling, kept):
    expected = np.zeros(len(LOGITS))
    expected[kept] = softmax([LOGITS[i] for i in kept])
    np.testing.assert_allclose(frequencies(sampling), expected, atol=0.015)
    # the inverse-CDF draw (an extension) samples the same distribution
    rng = np.random.default_rng(0)
    u = rng.random(20000, dtype=np.float32)
    got = oracle.sample(np.array([LOGITS] * 20000, np.float32), np.array([sampling], np.float32),
                        uniform_draws=u).ids.ravel()  # fmt: skip
    np.testing.assert_allclose(np.bincount(got, minlength=5) / 20000, expected, atol=0.015)


def test_top_p_zero_keeps_the_likeliest():
    rows = [LOGITS[::-1]] * 100
    assert set(draws(rows, values(1.0, top_p=0.0), list(range(100)), 0)) == {4}


def test_presence_penalty():
    seen = [[True, False, False, False, False]]
    assert draws([LOGITS], values(presence_penalty=1.5), 0, 0, seen) == [1]
    assert draws([LOGITS], values(presence_penalty=0.5), 0, 0, seen) == [0]


def test_seeded():
    flat = [[0.0] * 1000]
    first = draws(flat, values(1.0), 7, 3)
    assert draws(flat, values(1.0), 7, 3) == first
    assert draws(flat, values(1.0), 8, 3) != first and draws(flat, values(1.0), 7, 4) != first


def test_rows_are_their_own():
    ramp, peaked, flat = [i / 100 for i in range(1000)], LOGITS + [-9.0] * 995, [0.0] * 1000
    cut = values(1.0, top_k=10)
    alone = [draws([ramp], cut, 7, 3)[0], draws([peaked], values(), 0, 9)[0]]
    batched = draws([ramp, peaked, flat], [cut, values(), values(1.0)], [7, 0, 8], [3, 9, 5])
    assert batched[:2] == alone and batched[2] == draws([flat], values(1.0), 8, 5)[0]
    assert alone[0] >= 990


def test_hashed_uniform_is_a_23_bit_grid_inside_the_unit_interval():
    u = oracle.uniform([7, 8], [3, 4], 4096)
    assert u.dtype == np.float32 and u.min() >= 2.0**-24 and u.max() <= 1 - 2.0**-24
    assert (np.modf(u * 2.0**23)[0] == 0.5).all()
    # the value this restatement gave when it was first checked against the reference's formula
    np.testing.assert_array_equal(oracle.uniform([7], [3], 4)[0],
                                  np.array([0.82124513, 0.46080738, 0.9425561, 0.3054096], np.float32))  # fmt: skip


def test_hash_is_the_published_lowbias32():
    """leat's `_hash` (leat/sampler.py:67-73) is hash-prospector's lowbias32, a bijection of 32-bit
    words whose author also publishes its inverse (multipliers 0x43021123 and 0x1d69e2a5 with the
    shifts undone).  The published inverse, written out here independently, must take the hash back
    to its input, and its multipliers must be the forward ones' inverses modulo 2^32: that pins the
    restatement to the published function, not to itself."""
    assert (0x846CA68B * 0x43021123) % 2**32 == 1 and (0x7FEB352D * 0x1D69E2A5) % 2**32 == 1

    def inverse(x: int) -> int:
        x ^= x >> 16
        x = (x * 0x43021123) % 2**32
        x ^= (x >> 15) ^ (x >> 30)
        x = (x * 0x1D69E2A5) % 2**32
        x ^= x >> 16
        return x

    rng = np.random.default_rng(5)
    words = np.concatenate([np.array([0, 1, 2, 0xFFFFFFFF, 0x80000000, 0x7FFFFFFF], np.uint64),
                            rng.integers(0, 2**32, 2000, dtype=np.uint64)]).astype(np.uint32)  # fmt: skip
    hashed = oracle.lowbias32(words)
    assert hashed.dtype == np.uint32 and oracle.lowbias32(0)[0] == 0  # (zero is the hash's fixed point)
    assert [inverse(int(h)) for h in hashed] == [int(x) for x in words]
    assert len(set(hashed.tolist())) == len(set(words.tolist()))


@pytest.mark.parametrize("rows, n", [(1, 128256), (3, 1000), (2, 33), (1, 1)])
def test_argmax(rows, n):
    rng = np.random.default_rng(n)
    x = rng.integers(-50, 50, (rows, n)).astype(np.float32)
    x[:, ::7] = -np.inf
    np.testing.assert_array_equal(oracle.argmax(x), x.argmax(-1, keepdims=True))


@pytest.mark.parametrize("rows, n", [(1, 248320), (5, 32000), (2, 300)])
def test_cutoff_against_float64(rows, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal((rows, n)) * 2.5).astype(np.float32)
    x[:, : n // 100] += 9
    top_k, top_p = np.array([20, 0, 5, 1, 0][:rows]), np.array([0.95, 0.9, 1.0, 0.5, 0.0][:rows])
    for b in range(rows):
        ranked = -np.sort(-x[b])
        for order in ("sequential", "block"):
            c = oracle.cutoff_row(ranked, top_k[b], top_p[b], 0.0, order)
            top, by_k, by_p = oracle.cuts_f64(x[b], top_k[b], top_p[b])
            assert c.top == np.float32(top) and c.by_k == np.float32(by_k)
            # float32 running sums may tip a boundary by one rank; never by more than 1e-4 nat here
            assert abs(float(c.by_p) - by_p) <= 1e-4 or c.margin < 1e-5
    cut = oracle.cutoff(x, top_k.reshape(-1, 1), top_p.reshape(-1, 1), np.zeros((rows, 1)))
    assert cut.shape == (rows, 1)


def test_no_option_means_no_cut_and_min_p_floor():
    x = np.array([[3.0, 1.0, 2.0, -4.0]], np.float32)
    assert oracle.cutoff(x, [0], [1.0], [0.0])[0, 0] == -np.inf
    floor = oracle.cutoff(x, [0], [1.0], [0.5])[0, 0]
    assert floor == np.float32(3.0) + oracle.log32(np.float32(0.5))


def test_repetition_and_frequency_reduce_to_presence():
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((4, 500)).astype(np.float32) * 3
    history = rng.integers(0, 500, (4, 40)).astype(np.int32)
    seen = oracle.history_counts(history, None, 500) > 0
    options = np.array([[0.9, 20, 0.9, 0.0, 0.7]], np.float32)
    a = oracle.sample(logits, options, [5], 2, seen, keep_penalised=True)
    b = oracle.sample(logits, options, [5], 2, history=history, penalties=[[1.0, 0.7, 0.0]], keep_penalised=True)
    np.testing.assert_array_equal(a.penalised, b.penalised)
    np.testing.assert_array_equal(a.ids, b.ids)


def test_block_and_sequential_orders_agree_off_the_boundary():
    from leat_b200 import workloads

    w = workloads.config5(rows=48, vocab=20000)
    a = oracle.sample(w.logits, w.options, history=w.history, penalties=w.penalties, uniform_draws=w.uniform)
    b = oracle.sample(w.logits, w.options, history=w.history, penalties=w.penalties, uniform_draws=w.uniform,
                      order="block")  # fmt: skip
    differ = (a.ids != b.ids).ravel() | (a.kept != b.kept)
    assert (np.minimum(a.margin, b.margin)[differ] < 1e-5).all()
    np.testing.assert_array_equal(a.greedy, b.greedy)


def test_verify_draft():
    drafted = np.array([[5, 6, 7], [5, 6, 7], [1, 2, 3]], np.int32)
    sampled = np.array([[5, 6, 7, 8], [5, 9, 7, 8], [0, 2, 3, 4]], np.int32)
    kept, tokens = oracle.verify_draft(drafted, sampled)
    assert kept.tolist() == [3, 1, 0]
    assert tokens.tolist() == [[5, 6, 7, 8], [5, 9, -1, -1], [0, -1, -1, -1]]
    greedy = np.array([[5, 6, 0, 0], [5, 6, 7, 0], [9, 9, 9, 9]], np.int32)
    kept, tokens = oracle.verify_draft_greedy(drafted, greedy, sampled)
    assert kept.tolist() == [2, 3, 0]
    assert tokens.tolist() == [[5, 6, 7, -1], [5, 6, 7, 8], [0, -1, -1, -1]]
