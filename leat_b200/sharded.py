"""Vocabulary-sharded sampling: each rank holds a contiguous slice of every row's logits (a
tensor-parallel lm_head's layout), selects its slice's candidates on its own GPU, and one small
all-gather of (score, id) candidates per step lets every rank finish the same rows.  leat itself
has no multi-GPU path (one model per GPU, leat/server.py:427-428); the result is defined as the
single-GPU sampler's on the concatenated logits.

The two device steps are entry points of the CUDA library (leat_topk_local,
leat_sample_from_candidates); the exchange is torch.distributed (NCCL over NVLink on GPUs).
`select` and `finish` can be replaced for host-side tests of the exchange itself."""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from leat_b200 import _lib
from leat_b200.sampler import Sampled, Sampler, _stream
from leat_b200.workloads import shard_bounds


class ShardedSampler:
    """Samples rows whose vocabulary is split over the ranks of `group`.  `cap` is the number of
    candidates a rank may hand over per row (at least top_k plus room for ties)."""

    def __init__(self, max_rows: int, vocab: int, k_max: int = 64, cap: int | None = None, group=None,
                 device: torch.device | None = None, select=None, finish=None):  # fmt: skip
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.vocab = vocab
        self.start, self.stop = shard_bounds(vocab, self.world, self.rank)
        self.cap = cap or (k_max + 64)
        self.max_rows = max_rows
        self.device = device
        self._select, self._finish = select, finish
        self.sampler = None
        if select is None or finish is None:
            self.sampler = Sampler(max_rows, max(self.stop - self.start, 1), k_max, device)
            self.device = self.sampler.device
        d = self.device
        # what this rank hands over is one packed record (scores, ids, counts, greedy keys), so that
        # a single all-gather moves it; `all_records` is every rank's record, part-major
        if self.sampler is not None:
            size = _lib.lib.leat_candidate_record_bytes(max_rows, self.cap)
            at = [C.c_size_t(), C.c_size_t(), C.c_size_t()]
            _lib.check(_lib.lib.leat_candidate_record_layout(max_rows, self.cap, *(C.byref(x) for x in at)),
                       "leat_candidate_record_layout")  # fmt: skip
            id_at, count_at, best_at = (x.value for x in at)
        else:  # host-side stand-ins: the same layout, computed here
            values = max_rows * self.cap * 4
            id_at, count_at = values, 2 * values
            best_at = (2 * values + max_rows * 4 + 7) // 8 * 8
            size = (best_at + max_rows * 8 + 255) // 256 * 256
        self.record = torch.zeros(size, dtype=torch.uint8, device=d)
        self.all_records = torch.zeros(self.world * size, dtype=torch.uint8, device=d)
        rc = max_rows * self.cap

        def views(buffer, parts):
            per = buffer.view(parts, size)
            value = per[:, :id_at].view(torch.float32).view(parts, max_rows, self.cap)
            ids = per[:, id_at:count_at].view(torch.int32).view(parts, max_rows, self.cap)
            count = per[:, count_at:count_at + max_rows * 4].view(torch.int32).view(parts, max_rows)
            best = per[:, best_at:best_at + max_rows * 8].view(torch.int64).view(parts, max_rows)
            return value, ids, count, best

        value, ids, count, best = views(self.record, 1)
        self.value, self.ids, self.count, self.best = value[0], ids[0], count[0], best[0]
        self.all_value, self.all_ids, self.all_count, self.all_best = views(self.all_records, self.world)
        del rc

    # ---- the three steps ----------------------------------------------------------------------

    def select(self, logits_slice, options, seed, position, history=None, history_len=None,
               penalties=None, uniform=None, flags: int = 0) -> None:  # fmt: skip
        """This rank's candidates of its slice (rows, stop - start) into self.count/value/ids/best."""
        rows = logits_slice.shape[0]
        if rows > self.max_rows or logits_slice.shape[1] != self.stop - self.start:
            raise ValueError("logits_slice must be (rows <= max_rows, this rank's slice width)")
        if self._select is not None:
            self._select(self, logits_slice, options, seed, position, history, history_len, penalties, uniform)
            return
        a, keep = self.sampler._args(logits_slice, options, seed, position, None, history, history_len,
                                     penalties, uniform, flags, self.start, self.vocab)  # fmt: skip
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib.leat_topk_local(
                self.sampler.handle, C.byref(a), self.value.data_ptr(), self.ids.data_ptr(),
                self.count.data_ptr(), self.best.data_ptr(), self.cap, _stream()), "leat_topk_local")  # fmt: skip
        del keep

    def exchange(self, rows: int) -> None:
        """One all-gather: every rank ends with every rank's record, part-major."""
        if rows != self.max_rows:
            raise ValueError("the gather buffers are sized for max_rows rows")
        dist.all_gather_into_tensor(self.all_records, self.record, group=self.group)

    def finish(self, rows, options, seed, position, uniform=None, width: int = 0, flags: int = 0,
               out: torch.Tensor | None = None) -> Sampled:  # fmt: skip
        """Every rank finishes every row from the gathered candidates (the same result on all)."""
        if self._finish is not None:
            return self._finish(self, rows, options, seed, position, uniform, width)
        d = self.device
        dummy = torch.empty((rows, 4), dtype=torch.float32, device=d)  # shapes only: logits are not read
        a, keep = self.sampler._args(dummy, options, seed, position, None, None, None, None, uniform, flags)
        a.vocab, a.vocab_total = self.vocab, self.vocab
        ids = out if out is not None else torch.empty((rows, 1), dtype=torch.int32, device=d)
        result = Sampled(ids, status=torch.empty(1, dtype=torch.int32, device=d))  # cleared by the call (FLAG_CLEAR_STATUS)
        result.greedy = torch.empty(rows, dtype=torch.int32, device=d)
        result.cut = torch.empty(rows, dtype=torch.float32, device=d)
        result.kept = torch.empty(rows, dtype=torch.int32, device=d)
        a.out_ids, a.status = ids.data_ptr(), result.status.data_ptr()
        a.out_greedy, a.out_cut, a.out_kept = result.greedy.data_ptr(), result.cut.data_ptr(), result.kept.data_ptr()
        if width:
            result.probs = torch.empty((rows, width), dtype=torch.float32, device=d)
            result.prob_ids = torch.empty((rows, width), dtype=torch.int32, device=d)
            a.out_probs, a.out_prob_ids, a.out_width = result.probs.data_ptr(), result.prob_ids.data_ptr(), width
        with torch.cuda.device(d):
            _lib.check(_lib.lib.leat_sample_from_records(
                self.sampler.handle, C.byref(a), self.all_records.data_ptr(), self.world, self.cap, _stream()),
                "leat_sample_from_records")  # fmt: skip
        del keep
        return result

    def sample(self, logits_slice, options, seed=None, position=0, history=None, history_len=None,
               penalties=None, uniform=None, width: int = 0, flags: int = 0, out=None) -> Sampled:  # fmt: skip
        rows = logits_slice.shape[0]
        self.select(logits_slice, options, seed, position, history, history_len, penalties, uniform, flags)
        self.exchange(rows)
        return self.finish(rows, options, seed, position, uniform, width, flags, out)
