"""The tokens each cache slot's sequence has generated, kept as a short list of ids per slot instead
of leat's dense (slots, vocab) boolean mask (leat/engine.py:167-173).

leat marks a decode step's token in its slot's row of the mask with a (rows, vocab) one-hot pass
every step (`_generated`, leat/engine.py:768-781) and hands the sampler (rows, vocab) booleans,
which the sampler then reads in full.  Here a step appends one id per row, and the sampler gets
(rows, H) ids: B x H x 4 bytes instead of B x V.  As in leat, a format's markup tokens
(`tokenizer.special_ids`) are never recorded, a prompt chunk empties its slot, and recording a
token twice changes nothing for a presence penalty (it does count for the frequency penalty this
sampler adds).  A speculative step's rows see their slot's tokens plus the run's tokens up to their
own (`_seen_by`, leat/engine.py:664-675).

Everything is a handful of index operations on device tensors: no host synchronisation, fixed
shapes, so the calls can sit inside a captured CUDA graph.  It also runs on CPU tensors, which is
how its logic is tested without a GPU."""

from __future__ import annotations

import torch


class SlotHistory:
    """ids (slots, capacity) int32 with -1 for unused places (the sampler ignores ids outside the
    vocabulary), count (slots,) int32 of tokens recorded so far; a slot's list is a ring: once
    `capacity` tokens are in, the oldest are overwritten."""

    def __init__(self, slots: int, capacity: int, vocab: int, special_ids=(), device=None):
        if slots <= 0 or capacity <= 0 or vocab <= 0:
            raise ValueError("slots, capacity and vocab must be positive")
        self.slots, self.capacity, self.vocab = slots, capacity, vocab
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.ids = torch.full((slots, capacity), -1, dtype=torch.int32, device=self.device)
        self.count = torch.zeros(slots, dtype=torch.int32, device=self.device)
        text = torch.ones(vocab, dtype=torch.bool)
        special = [i for i in special_ids if 0 <= i < vocab]
        if special:
            text[torch.tensor(special, dtype=torch.long)] = False
        self.text = text.to(self.device)  # leat's `_text`: tokens a penalty may lower

    def reset(self, slots: torch.Tensor) -> None:
        """A chunk of prompt empties its slot's tokens (leat/engine.py:772-774)."""
        slots = slots.to(self.device, torch.long).reshape(-1)
        self.ids[slots] = -1
        self.count[slots] = 0

    def append(self, slots: torch.Tensor, tokens: torch.Tensor) -> None:
        """A decode step runs its rows' last tokens and adds each to its slot's (rows with distinct
        slots), unless the token is markup."""
        slots = slots.to(self.device, torch.long).reshape(-1)
        tokens = tokens.to(self.device, torch.long).reshape(-1)
        keep = self.text[tokens.clamp(0, self.vocab - 1)] & (tokens >= 0) & (tokens < self.vocab)
        count = self.count[slots].to(torch.long)
        place = count % self.capacity
        old = self.ids[slots, place]
        self.ids[slots, place] = torch.where(keep, tokens.to(torch.int32), old)
        self.count[slots] = (count + keep.to(torch.long)).to(torch.int32)

    def rows(self, slots: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(history, history_len) for a decode step over `slots`: what sample() takes."""
        slots = slots.to(self.device, torch.long).reshape(-1)
        return self.ids[slots].contiguous(), self.count[slots].clamp(max=self.capacity).contiguous()

    def rows_of_run(self, slots: torch.Tensor, run: torch.Tensor) -> torch.Tensor:
        """History of a speculative step's rows: `run` (n, ran) are the tokens each sequence runs; row
        (i, j) sees its slot's tokens and run tokens 0..j, markup left out.  Returns
        (n * ran, capacity + ran) ids, -1 where nothing is recorded (no lengths needed)."""
        slots = slots.to(self.device, torch.long).reshape(-1)
        run = run.to(self.device, torch.long)
        n, ran = run.shape
        base = self.ids[slots].unsqueeze(1).expand(n, ran, self.capacity)
        ok = self.text[run.clamp(0, self.vocab - 1)] & (run >= 0) & (run < self.vocab)
        shown = torch.where(ok, run, torch.full_like(run, -1)).to(torch.int32)  # (n, ran)
        upto = torch.tril(torch.ones(ran, ran, dtype=torch.bool, device=self.device))  # row j sees tokens 0..j
        tail = torch.where(upto.unsqueeze(0), shown.unsqueeze(1).expand(n, ran, ran), torch.full((), -1, dtype=torch.int32, device=self.device))
        return torch.cat([base, tail], dim=2).reshape(n * ran, self.capacity + ran).contiguous()

    def dense(self, slots: torch.Tensor) -> torch.Tensor:
        """The (rows, vocab) boolean mask leat would hold for these slots (for tests and for callers
        that still want it)."""
        ids, length = self.rows(slots)
        return dense_mask(ids, self.vocab, length)


def dense_mask(ids: torch.Tensor, vocab: int, length: torch.Tensor | None = None) -> torch.Tensor:
    """(rows, vocab) booleans from (rows, H) ids; ids outside [0, vocab) and places at or beyond
    `length` count for nothing."""
    rows, width = ids.shape
    ids = ids.to(torch.long)
    valid = (ids >= 0) & (ids < vocab)
    if length is not None:
        valid &= torch.arange(width, device=ids.device).unsqueeze(0) < length.to(torch.long).unsqueeze(1)
    mask = torch.zeros((rows, vocab + 1), dtype=torch.bool, device=ids.device)
    mask.scatter_(1, torch.where(valid, ids, torch.full_like(ids, vocab)), True)
    return mask[:, :vocab].contiguous()


def options_row(sampling, frequency_penalty: float = 0.0, repetition_penalty: float = 1.0) -> tuple[list[float], list[float]]:
    """A request's sampling settings as the two rows the sampler reads: options
    (temperature, top_k, top_p, min_p, presence_penalty), as `Sampling.values()` lays them out
    (leat/sampler.py:17-25, used at leat/engine.py:569), and penalties (repetition, presence,
    frequency), which also carries the two penalties leat's server refuses today
    (leat/server.py:84-115)."""
    options = [float(v) for v in sampling.values()]
    return options, [float(repetition_penalty), float(sampling.presence_penalty), float(frequency_penalty)]
