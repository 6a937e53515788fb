"""The host side of vocabulary-sharded sampling on two gloo ranks (CPU): slice bounds, the layout
of what is gathered, and that finishing from the gathered candidates gives the single-device
result.  The two device steps are replaced by CPU stand-ins built on the oracle, so this checks the
plumbing of leat_b200/sharded.py, not the kernels (those are checked on GPUs)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from leat_b200 import workloads
from oracle import sampler_oracle as oracle

ROWS, VOCAB, CAP = 6, 4000, 96


def _select(self, logits_slice, options, seed, position, history, history_len, penalties, uniform):
    count, values, ids, best, best_id = oracle.local_candidates(
        logits_slice.numpy(), options.numpy(), self.start, self.cap,
        history=None if history is None else history.numpy(),
        penalties=None if penalties is None else penalties.numpy())  # fmt: skip
    self.count.copy_(torch.from_numpy(count))
    self.value.copy_(torch.from_numpy(values))
    self.ids.copy_(torch.from_numpy(ids))
    packed = (best.view(np.uint32).astype(np.int64) << 32) | best_id.astype(np.int64)
    self.best.copy_(torch.from_numpy(packed))


def _finish(self, rows, options, seed, position, uniform, width):
    # scores of the gathered candidates on an otherwise empty vocabulary, sampled at temperature 1
    scores = np.full((rows, self.vocab), -np.inf, np.float32)
    counts, values, ids = self.all_count.numpy(), self.all_value.numpy(), self.all_ids.numpy()
    for part in range(self.world):
        for b in range(rows):
            n = counts[part, b]
            assert 0 <= n <= self.cap
            scores[b, ids[part, b, :n]] = values[part, b, :n]
    opts = options.numpy().copy()
    greedy_rows = opts[:, 0] <= 0
    opts[:, 0] = 1.0
    out = oracle.sample(scores, opts, uniform_draws=uniform.numpy(), scale="divide")
    best = self.all_best.numpy()
    greedy_ids = np.array([int(best[np.argmax(best[:, b] >> 32), b] & 0xFFFFFFFF) for b in range(rows)])
    out.ids[greedy_rows, 0] = greedy_ids[greedy_rows]
    return out


def _rank(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from leat_b200.sharded import ShardedSampler

        w = workloads.config5(rows=ROWS, vocab=VOCAB)
        w.options[1, 0] = 0.0  # one greedy row
        sharded = ShardedSampler(ROWS, VOCAB, k_max=64, cap=CAP, device=torch.device("cpu"), select=_select, finish=_finish)
        start, stop = sharded.start, sharded.stop
        assert (start, stop) == workloads.shard_bounds(VOCAB, world, rank)
        t = torch.from_numpy
        out = sharded.sample(t(np.ascontiguousarray(w.logits[:, start:stop])), t(w.options), None, 0,
                             history=t(w.history), penalties=t(w.penalties), uniform=t(w.uniform))  # fmt: skip
        assert tuple(sharded.all_value.shape) == (world, ROWS, CAP)
        # what was gathered from this rank is what this rank selected
        assert torch.equal(sharded.all_count[rank], sharded.count)
        assert torch.equal(sharded.all_ids[rank], sharded.ids)
        results[rank] = (out.ids.ravel().tolist(), out.kept.tolist())
    finally:
        dist.destroy_process_group()


def test_two_ranks_agree_with_one_device():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, port, results), nprocs=2, join=True)
    w = workloads.config5(rows=ROWS, vocab=VOCAB)
    w.options[1, 0] = 0.0
    whole = oracle.sample(w.logits, w.options, history=w.history, penalties=w.penalties, uniform_draws=w.uniform)
    assert results[0] == results[1]
    ids, kept = results[0]
    firm = whole.margin >= 1e-5
    assert (np.array(ids)[firm] == whole.ids.ravel()[firm]).all()
    sampled = firm & (w.options[:, 0] > 0)
    assert (np.array(kept)[sampled] == whole.kept[sampled]).all()
