"""GPU parity of the peer-exchange shards (leat_shard_select / leat_shard_finish / leat_shard_result),
emulated on one GPU: the N ranks are N shard objects of one process whose exchange regions are plain
device allocations every "rank" can address.  The three phases of a step run rank after rank, phase
after phase, on one stream, so that no kernel ever waits for a kernel launched after it; every
rank's results must be the same and equal the oracle's on the whole vocabulary."""

import ctypes as C

import numpy as np
import pytest

from tests import helpers

pytestmark = pytest.mark.gpu


class PeerShardsOnOneGpu:
    def __init__(self, device, rows, vocab, parts, cap=128, k_max=64):
        import torch

        from leat_b200 import _lib, workloads
        from leat_b200.sampler import Sampler

        self.device, self.rows, self.vocab, self.parts, self.cap = device, rows, vocab, parts, cap
        self.bounds = [workloads.shard_bounds(vocab, parts, r) for r in range(parts)]
        self.samplers = [Sampler(rows, max(b - a, 8), k_max, device) for a, b in self.bounds]
        size = _lib.lib.leat_shard_region_bytes(rows, cap, parts)
        assert size > 0
        self.regions = [torch.zeros(size + 256, dtype=torch.uint8, device=device) for _ in range(parts)]
        bases = [(r.data_ptr() + 255) // 256 * 256 for r in self.regions]
        self.shards = []
        for rank in range(parts):
            shard = C.c_void_p()
            _lib.check(_lib.lib.leat_shard_create(self.samplers[rank].handle, rank, parts, rows, cap,
                                                  (C.c_void_p * parts)(*bases), C.byref(shard)), "leat_shard_create")  # fmt: skip
            self.shards.append(shard)
        torch.cuda.synchronize()

    def close(self):
        from leat_b200 import _lib

        for shard in self.shards:
            _lib.lib.leat_shard_destroy(shard)

    def step(self, w, mode, leave_out=None, dtype=None):
        """One step of every rank; returns each rank's Sampled.  `leave_out`: a rank that does not
        take the step at all (the others must notice, not hang); `dtype`: the slices' format on the
        device, if not float32."""
        import torch

        from leat_b200 import _lib
        from leat_b200.sampler import Sampled, _stream

        d = self.device
        t = lambda x: None if x is None else torch.as_tensor(x).to(d)  # noqa: E731
        seed = torch.as_tensor(w.seed.astype(np.int64)).to(d).to(torch.uint32)
        options, penalties, history, position = t(w.options), t(w.penalties), t(w.history), t(w.position)
        uniform = t(w.uniform) if mode == "U" else None
        ranks = [r for r in range(self.parts) if r != leave_out]
        calls, results, keeps = {}, {}, []
        for r in ranks:
            start, stop = self.bounds[r]
            part = torch.as_tensor(np.ascontiguousarray(w.logits[:, start:stop])).to(d)
            part = part if dtype is None else part.to(dtype)
            a, keep = self.samplers[r]._args(part, options, seed, position, None, history, None, penalties, uniform,
                                             0, start, self.vocab)  # fmt: skip
            out = Sampled(torch.empty((self.rows, 1), dtype=torch.int32, device=d),
                          status=torch.empty(1, dtype=torch.int32, device=d))  # fmt: skip
            out.greedy = torch.empty(self.rows, dtype=torch.int32, device=d)
            out.cut = torch.empty(self.rows, dtype=torch.float32, device=d)
            out.kept = torch.empty(self.rows, dtype=torch.int32, device=d)
            a.status = out.status.data_ptr()
            calls[r], results[r] = a, out
            keeps.append((part, keep))
            _lib.check(_lib.lib.leat_shard_select(self.shards[r], C.byref(a), _stream()), "leat_shard_select")
        for r in ranks:
            a, out = calls[r], results[r]
            a.logits, a.vocab, a.vocab_total, a.vocab_offset = None, self.vocab, self.vocab, 0
            a.history, a.history_len, a.history_cap, a.penalties, a.penalties_rows = None, None, 0, None, 0
            a.flags &= ~_lib.FLAG_CLEAR_STATUS
            a.out_ids, a.out_greedy = out.ids.data_ptr(), out.greedy.data_ptr()
            a.out_cut, a.out_kept = out.cut.data_ptr(), out.kept.data_ptr()
            _lib.check(_lib.lib.leat_shard_finish(self.shards[r], C.byref(a), _stream()), "leat_shard_finish")
        for r in ranks:
            _lib.check(_lib.lib.leat_shard_result(self.shards[r], C.byref(calls[r]), _stream()), "leat_shard_result")
        torch.cuda.synchronize()
        del keeps
        return results


def _workload(rows=24, vocab=201088):
    from leat_b200 import workloads

    w = workloads.config5(rows=rows, vocab=vocab)
    w.options[3, 0] = 0.0  # a greedy row among them
    w.options[5, 1:4] = (0.0, 1.0, 0.02)  # min-p alone
    w.options[7, 1] = 20.0  # another top_k
    return w


@pytest.mark.parametrize("parts", [2, 4, 8])
@pytest.mark.parametrize("mode", ["U", "G"])
def test_peer_shards_equal_the_single_device_oracle(device, parts, mode):
    w = _workload()
    emu = PeerShardsOnOneGpu(device, w.rows, w.vocab, parts)
    try:
        want = helpers.oracle_run(w, mode)
        for step in range(3):  # both parities of the exchange buffers, and a buffer's second use
            results = emu.step(w, mode)
            for r, got in results.items():
                assert int(got.status.item()) & 12 == 0, f"rank {r}: status {int(got.status.item())}"
                helpers.compare(want, got, 0, max_fragile=1)
                np.testing.assert_array_equal(got.kept.cpu().numpy()[w.options[:, 0] > 0], want.kept[w.options[:, 0] > 0])
                np.testing.assert_array_equal(got.ids.cpu().numpy(), results[0].ids.cpu().numpy())
    finally:
        emu.close()


def test_peer_shards_on_slices_too_narrow_to_filter(device):
    """Slices under 16384 tokens are streamed by sample_kernel, which hands the rows over itself."""
    w = _workload(rows=10, vocab=50048)
    w.options[2, 1:4] = (0.0, 1.0, 0.0)  # no cut at all: whole-row hashed draw
    emu = PeerShardsOnOneGpu(device, w.rows, w.vocab, 4)
    try:
        for mode in ("G", "U"):
            if mode == "U":
                w.options[2, 1] = 30.0  # (the supplied-uniform draw with no cut is the multi-pass routine's)
            want = helpers.oracle_run(w, mode)
            for r, got in emu.step(w, mode).items():
                assert int(got.status.item()) & 12 == 0
                helpers.compare(want, got, 0, max_fragile=1)
    finally:
        emu.close()


def test_a_rank_that_never_takes_the_step_is_noticed(device):
    """Failure detection without a fault: one rank skips the step, so its hand-overs never arrive;
    the other ranks' waits run out (about a second), their kernels end, the status word carries
    LEAT_STATUS_PEER and the ids read -1.  Nothing hangs and the context stays usable."""
    import torch

    from leat_b200 import _lib

    w = _workload(rows=8, vocab=70000)
    emu = PeerShardsOnOneGpu(device, w.rows, w.vocab, 2)
    try:
        results = emu.step(w, "U", leave_out=1)
        got = results[0]
        assert int(got.status.item()) & _lib.STATUS_PEER
        assert (got.ids.cpu().numpy() == -1).all()
        assert float(torch.ones(4, device=device).sum().item()) == 4.0  # the device still answers
    finally:
        emu.close()
