"""The reference's own sampler tests (leat tests/test_sampler.py:37-93 and the argmax / cutoff
kernel tests of tests/test_kernels.py:927-955) run against the CUDA library through the Python
face, which calls the C ABI."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LOGITS = [2.0, 1.0, 0.0, -1.0, 0.5]


@pytest.fixture(scope="module")
def api(device):
    import torch

    from leat_b200 import ops
    from leat_b200.sampler import Sampling, sample

    def draws(logits, sampling, seed, position, seen=None):
        options = torch.tensor([s.values() for s in (sampling if isinstance(sampling, list) else [sampling])],
                               dtype=torch.float32, device=device)  # fmt: skip
        seeds = torch.tensor(seed if isinstance(seed, list) else [seed], dtype=torch.int64).to(device).to(torch.uint32)
        positions = torch.tensor(position, dtype=torch.int32, device=device) if isinstance(position, list) else position
        marked = None if seen is None else torch.tensor(seen, dtype=torch.bool, device=device)
        out = sample(torch.tensor(logits, dtype=torch.float32, device=device), options, seeds, positions, marked)
        assert out.dtype == torch.int32 and tuple(out.shape) == (len(logits), 1) and out.is_cuda
        return out.cpu().numpy().ravel().tolist()

    return draws, Sampling, ops


def frequencies(draws, sampling, n=20000, rows=1000):
    got = [t for i in range(0, n, rows) for t in draws([LOGITS] * rows, sampling, list(range(i, i + rows)), 0)]
    return np.bincount(got, minlength=len(LOGITS)) / n


def softmax(logits, temperature=1.0):
    p = np.exp(np.array(logits) / temperature)
    return p / p.sum()


def test_greedy(api):
    draws, Sampling, _ = api
    assert draws([LOGITS, LOGITS[::-1]], Sampling(), 0, 0) == [0, 4]


def test_temperature_matches_softmax(api):
    draws, Sampling, _ = api
    np.testing.assert_allclose(frequencies(draws, Sampling(0.7)), softmax(LOGITS, 0.7), atol=0.015)


@pytest.mark.parametrize("options, kept", [
    (dict(top_k=2), [0, 1]),
    (dict(top_k=4, top_p=0.8), [0, 1, 4]),
    (dict(top_p=0.5), [0]),
    (dict(min_p=0.2), [0, 1, 4]),
])  # fmt: skip
def test_cut_tokens_never_drawn(api, options, kept):
    draws, Sampling, _ = api
    expected = np.zeros(len(LOGITS))
    expected[kept] = softmax([LOGITS[i] for i in kept])
    np.testing.assert_allclose(frequencies(draws, Sampling(1.0, **options)), expected, atol=0.015)


def test_top_p_zero_keeps_the_likeliest(api):
    draws, Sampling, _ = api
    rows = [LOGITS[::-1]] * 100
    assert set(draws(rows, Sampling(1.0, top_p=0.0), list(range(100)), 0)) == {4}


def test_presence_penalty(api):
    draws, Sampling, _ = api
    seen = [[True, False, False, False, False]]
    assert draws([LOGITS], Sampling(presence_penalty=1.5), 0, 0, seen) == [1]
    assert draws([LOGITS], Sampling(presence_penalty=0.5), 0, 0, seen) == [0]


def test_seeded(api):
    draws, Sampling, _ = api
    flat = [[0.0] * 1000]
    first = draws(flat, Sampling(1.0), 7, 3)
    assert draws(flat, Sampling(1.0), 7, 3) == first
    assert draws(flat, Sampling(1.0), 8, 3) != first and draws(flat, Sampling(1.0), 7, 4) != first


def test_rows_are_their_own(api):
    draws, Sampling, _ = api
    ramp, peaked, flat = [i / 100 for i in range(1000)], LOGITS + [-9.0] * 995, [0.0] * 1000
    cut = Sampling(1.0, top_k=10)
    alone = [draws([ramp], cut, 7, 3)[0], draws([peaked], Sampling(), 0, 9)[0]]
    batched = draws([ramp, peaked, flat], [cut, Sampling(), Sampling(1.0)], [7, 0, 8], [3, 9, 5])
    assert batched[:2] == alone and batched[2] == draws([flat], Sampling(1.0), 8, 5)[0]
    assert alone[0] >= 990


def test_draws_equal_the_oracle(api):
    # the hashed Gumbel draw, id for id, on the rows the reference's tests use
    from oracle import sampler_oracle as oracle

    draws, Sampling, _ = api
    for sampling in (Sampling(0.7), Sampling(1.0, top_k=2), Sampling(1.0, top_k=4, top_p=0.8), Sampling(1.0, min_p=0.2)):
        seeds = list(range(500))
        got = draws([LOGITS] * 500, sampling, seeds, 11)
        want = oracle.sample(np.array([LOGITS] * 500, np.float32), np.array([sampling.values()], np.float32),
                             np.array(seeds, np.uint32), 11, order="block")  # fmt: skip
        differ = np.nonzero(np.array(got) != want.ids.ravel())[0]
        assert (want.margin[differ] < 1e-5).all() and len(differ) <= 2


@pytest.mark.parametrize("rows, n", [(1, 128256), (3, 1000), (2, 33), (1, 1), (5, 151936), (300, 16384), (4, 262144),
                                     (700, 4096), (2, 4100)])  # fmt: skip
def test_argmax(api, device, rows, n):
    """Rows of whole aligned vectors take the one-launch kernel, the others the sampler's greedy path."""
    import torch

    _, _, ops = api
    rng = np.random.default_rng(n)
    x = rng.integers(-50, 50, (rows, n)).astype(np.float32)  # many ties: the first one must win
    x[:, ::7] = -np.inf
    x[-1, :] = -np.inf  # a row of nothing but -inf answers 0
    if rows > 1:
        x[0, : n // 2] = -np.inf  # the maximum lies in a later span
        x[0, n - 1] = 60.0  # ... at the row's very end
    got = ops.argmax(torch.tensor(x, device=device))
    assert got.dtype == torch.int32
    np.testing.assert_array_equal(got.cpu().numpy(), x.argmax(-1, keepdims=True))
