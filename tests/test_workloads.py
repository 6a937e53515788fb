"""Host logic: the synthetic workloads are deterministic and shaped as the configurations say, and
vocabulary slices tile the vocabulary."""

import numpy as np

from leat_b200 import workloads


def test_workloads_are_seeded_and_shaped():
    a, b = workloads.config2(rows=4, vocab=4096), workloads.config2(rows=4, vocab=4096)
    np.testing.assert_array_equal(a.logits, b.logits)
    np.testing.assert_array_equal(a.history, b.history)
    assert a.logits.dtype == np.float32 and a.history.shape == (4, 1024) and a.options.shape == (4, 5)
    assert (a.logits == 12.0).sum(axis=1).tolist() == [5] * 4
    c3 = workloads.config3(rows=16, vocab=8192)
    assert (c3.options[:, 0] == 0).sum() == 4 and c3.history.shape == (16, 2048)
    c4 = workloads.config4(sequences=2, vocab=4096)
    assert c4.logits.shape == (18, 4096) and c4.drafted.shape == (2, 8)
    assert {n: workloads.SHAPES[n] for n in (1, 3, 5)} == {1: (1, 128256), 3: (256, 262144), 5: (512, 201088)}


def test_shard_bounds_tile_the_vocabulary():
    for vocab in (201088, 128256, 1000, 7):
        for parts in (1, 2, 4, 8):
            edges = [workloads.shard_bounds(vocab, parts, r) for r in range(parts)]
            assert edges[0][0] == 0 and edges[-1][1] == vocab
            assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
            assert all(start % 4 == 0 for start, stop in edges if stop > start)
