"""Vocabulary-sharded sampling: each rank holds a contiguous slice of every row's logits (a
tensor-parallel lm_head's layout), selects its slice's candidates on its own GPU, and one small
exchange of (score, id) candidates per step lets the ranks finish the rows.  leat itself has no
multi-GPU path (one model per GPU, leat/server.py:427-428); the result is defined as the
single-GPU sampler's on the concatenated logits.

Two exchanges:

* "peer" (GPUs of one node): every rank owns a share of the rows.  The select kernels store each
  row's candidates straight into the owning rank's exchange region over NVLink (plain stores to
  peer-mapped memory), the owner finishes its rows and stores the results into every rank's region;
  flags carrying the step number order it all, every wait is bounded, and no collective is called
  (leat_shard_select / leat_shard_finish / leat_shard_result of the CUDA library).  A whole step is
  a handful of kernel launches that can be captured in one CUDA graph.
* "collective": one all-gather of packed candidate records (torch.distributed; NCCL on GPUs, gloo
  in the CPU tests), then every rank finishes every row (leat_topk_local,
  leat_sample_from_records).  `select` and `finish` can be replaced for host-side tests of the
  exchange itself.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from leat_b200 import _lib
from leat_b200.sampler import Sampled, Sampler, _stream
from leat_b200.workloads import shard_bounds


class ShardedSampler:
    """Samples rows whose vocabulary is split over the ranks of `group`.  `cap` is the number of
    candidates a rank may hand over per row (at least top_k plus room for ties).  `exchange` is
    "peer", "collective" or "auto" (peer where the ranks' regions can be mapped into one another,
    which all ranks agree on; else collective)."""

    def __init__(self, max_rows: int, vocab: int, k_max: int = 64, cap: int | None = None, group=None,
                 device: torch.device | None = None, select=None, finish=None, exchange: str = "auto"):  # fmt: skip
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
        self.shard = None
        self._regions: list[int] = []
        self._opened: list[int] = []
        if select is None or finish is None:
            self.sampler = Sampler(max_rows, max(self.stop - self.start, 1), k_max, device)
            self.device = self.sampler.device
        if exchange not in ("auto", "peer", "collective"):
            raise ValueError("exchange must be 'auto', 'peer' or 'collective'")
        self.exchange_kind = "collective"
        if exchange != "collective" and self.sampler is not None and self.world <= 8:
            if self._open_peer_exchange():
                self.exchange_kind = "peer"
            elif exchange == "peer":
                raise RuntimeError("the ranks' exchange regions could not be mapped into one another")
        elif exchange == "peer":
            raise RuntimeError("the peer exchange needs the CUDA library and at most 8 ranks")
        if self.exchange_kind == "collective":
            self._make_records()

    # ---- the peer exchange ----------------------------------------------------------------------

    def _open_peer_exchange(self) -> bool:
        """Allocates this rank's exchange region, maps every other rank's, and builds the library's
        shard object.  False (on every rank alike) if any rank could not."""
        size = _lib.lib.leat_shard_region_bytes(self.max_rows, self.cap, self.world)
        own, handle = C.c_void_p(), C.create_string_buffer(64)
        ok = size > 0
        with torch.cuda.device(self.device):
            ok = ok and _lib.lib.leat_peer_alloc(size, C.byref(own), handle) == _lib.OK
            mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device=self.device)
            everyone = torch.zeros(self.world * 64, dtype=torch.uint8, device=self.device)
            dist.all_gather_into_tensor(everyone, mine, group=self.group)
            handles = everyone.cpu().numpy().tobytes()
            regions = []
            for r in range(self.world):
                if r == self.rank:
                    regions.append(own.value)
                    continue
                ptr = C.c_void_p()
                if ok and _lib.lib.leat_peer_open(handles[64 * r: 64 * r + 64], C.byref(ptr)) == _lib.OK:
                    self._opened.append(ptr.value)
                    regions.append(ptr.value)
                else:
                    ok = False
                    regions.append(None)
            agreed = torch.tensor([int(bool(ok))], dtype=torch.int32, device=self.device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)  # (also: every region is zeroed by now)
            if not int(agreed.item()):
                self._close_peer_exchange(own.value)
                return False
            self._own_region = own.value
            self._regions = regions
            shard = C.c_void_p()
            _lib.check(_lib.lib.leat_shard_create(self.sampler.handle, self.rank, self.world, self.max_rows, self.cap,
                                                  (C.c_void_p * self.world)(*regions), C.byref(shard)), "leat_shard_create")  # fmt: skip
            self.shard = shard
            dist.barrier(group=self.group)
        return True

    def _close_peer_exchange(self, own) -> None:
        for ptr in self._opened:
            _lib.lib.leat_peer_close(ptr)
        self._opened = []
        if own:
            _lib.lib.leat_peer_free(own)

    def close(self) -> None:
        """Frees the peer exchange (every rank, after its last step has finished on the device)."""
        if self.shard is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # nobody stores into a region that is going away
            _lib.lib.leat_shard_destroy(self.shard)
            self.shard = None
            self._close_peer_exchange(self._own_region)

    def _peer_step(self, logits_slice, options, seed, position, history, history_len, penalties, uniform, flags, out):
        rows = logits_slice.shape[0]
        if rows != self.max_rows:
            raise ValueError("the exchange regions are sized for max_rows rows")
        d = self.device
        a, keep = self.sampler._args(logits_slice, options, seed, position, None, history, history_len,
                                     penalties, uniform, flags, self.start, self.vocab)  # fmt: skip
        ids = out if out is not None else torch.empty((rows, 1), dtype=torch.int32, device=d)
        result = Sampled(ids, status=torch.empty(1, dtype=torch.int32, device=d))  # cleared by the select (FLAG_CLEAR_STATUS)
        result.greedy = torch.empty(rows, dtype=torch.int32, device=d)
        result.cut = torch.empty(rows, dtype=torch.float32, device=d)
        result.kept = torch.empty(rows, dtype=torch.int32, device=d)
        a.status = result.status.data_ptr()
        with torch.cuda.device(d):
            _lib.check(_lib.lib.leat_shard_select(self.shard, C.byref(a), _stream()), "leat_shard_select")
            a.logits, a.vocab, a.vocab_total, a.vocab_offset = None, self.vocab, self.vocab, 0
            a.history, a.history_len, a.history_cap, a.penalties, a.penalties_rows = None, None, 0, None, 0
            a.flags &= ~_lib.FLAG_CLEAR_STATUS
            a.out_ids, a.out_greedy = ids.data_ptr(), result.greedy.data_ptr()
            a.out_cut, a.out_kept = result.cut.data_ptr(), result.kept.data_ptr()
            _lib.check(_lib.lib.leat_shard_finish(self.shard, C.byref(a), _stream()), "leat_shard_finish")
            _lib.check(_lib.lib.leat_shard_result(self.shard, C.byref(a), _stream()), "leat_shard_result")
        del keep
        return result

    # ---- the collective exchange -----------------------------------------------------------------

    def _make_records(self) -> None:
        d, max_rows = self.device, self.max_rows
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

    # ---- a step -----------------------------------------------------------------------------------

    def sample(self, logits_slice, options, seed=None, position=0, history=None, history_len=None,
               penalties=None, uniform=None, width: int = 0, flags: int = 0, out=None) -> Sampled:  # fmt: skip
        """One step on this rank's slice; ids, greedy ids, cuts and survivor counts of all rows, the
        same on every rank.  (Probabilities, `width`, come with the collective exchange only.)"""
        if self.exchange_kind == "peer":
            if width:
                raise ValueError("the peer exchange does not return probabilities")
            return self._peer_step(logits_slice, options, seed, position, history, history_len, penalties, uniform, flags, out)
        rows = logits_slice.shape[0]
        self.select(logits_slice, options, seed, position, history, history_len, penalties, uniform, flags)
        self.exchange(rows)
        return self.finish(rows, options, seed, position, uniform, width, flags, out)

    @property
    def exchange_note(self) -> str:
        if self.exchange_kind == "peer":
            return ("peer memory: each row's candidates stored into its owning rank's region over NVLink, "
                    "results stored back into every rank's; flags with bounded waits, no collective")
        return "one all-gather of packed (score, id, count, greedy) candidate records per step, every rank finishes every row"

    @property
    def launches_per_step(self) -> int:
        """Kernels of this library a step launches on a rank: filter, select, streaming pass, finish,
        results (peer); filter, candidates, second pass, finish (collective)."""
        return 5 if self.exchange_kind == "peer" else 4

    def replayable(self, pool, options, seed, position, history, penalties, uniform, out, per_graph: int = 1):
        """A function replay(i) that runs `per_graph` consecutive steps (over pool[0], pool[1], ...
        in turn) from captured CUDA graphs, as a serving engine that replays captured decode steps
        would, and a sentence saying how.  With the peer exchange the steps are one graph; with the
        collective one, each step's two device steps are graphs and the all-gather is issued between
        them."""
        rows = pool[0].shape[0]
        side = torch.cuda.Stream()
        if self.exchange_kind == "peer":
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for j in range(per_graph):
                        self.sample(pool[j % len(pool)], options, seed, position, history=history, penalties=penalties,
                                    uniform=uniform, out=out)  # fmt: skip
            torch.cuda.synchronize()
            return (lambda i: graph.replay()), f"every replay is one CUDA graph holding {per_graph} whole steps"
        selects, finish = [], torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for buffer in pool:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self.select(buffer, options, seed, position, history, None, penalties, uniform)
                selects.append(g)
            with torch.cuda.graph(finish, stream=side):
                self.finish(rows, options, seed, position, uniform, out=out)
        torch.cuda.synchronize()

        def replay(i):
            for j in range(per_graph):
                selects[j % len(selects)].replay()
                self.exchange(rows)
                finish.replay()

        return replay, "the two device steps replayed from CUDA graphs, the all-gather issued eagerly between them"
