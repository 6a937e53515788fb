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


# what each option must be, as leat's server and defaults state it (leat/server.py:84-109: temperature
# 0..2, top_k an integer, top_p and min_p 0..1, presence_penalty -2..2; leat/defaults.py:26-29: top_k up
# to 2^20), and the ranges this sampler gives the two penalties leat's server refuses outright
# (leat/server.py:112-115): OpenAI's -2..2 for frequency_penalty, (0, 2] for repetition_penalty
BOUNDS = {
    "temperature": (0.0, 2.0), "top_k": (0, 1 << 20), "top_p": (0.0, 1.0), "min_p": (0.0, 1.0),
    "presence_penalty": (-2.0, 2.0), "frequency_penalty": (-2.0, 2.0), "repetition_penalty": (0.0, 2.0),
}  # fmt: skip


def _number(name: str, value, integer: bool = False) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value:
        raise ValueError(f"{name} must be {'an integer' if integer else 'a number'}")
    if integer and int(value) != value:
        raise ValueError(f"{name} must be an integer")
    return value


def sampling_from_request(body: dict, defaults: dict | None = None):
    """A request's sampling fields as a `Sampling` plus the two extra penalties, checked as leat's
    server checks them (leat/server.py:84-109, :921-924): a field that is absent or None takes the
    default (OpenAI's, leat/defaults.py:31, unless `defaults` says otherwise), a top_k of -1 (vLLM's
    "every token") becomes 0, and a value outside its range raises ValueError.  Returns
    (Sampling, frequency_penalty, repetition_penalty)."""
    from leat_b200.sampler import Sampling

    base = {"temperature": 1.0, "top_k": 0, "top_p": 1.0, "min_p": 0.0, "presence_penalty": 0.0}
    base.update(defaults or {})
    given = {k: v for k, v in body.items() if v is not None}
    values = {}
    for name in ("temperature", "top_k", "top_p", "min_p", "presence_penalty"):
        value = _number(name, given.get(name, base[name]), integer=name == "top_k")
        if name == "top_k":
            value = max(int(value), 0)  # vLLM's -1: every one
        low, high = BOUNDS[name]
        if not low <= value <= high:
            raise ValueError(f"{name} must be a number from {low} to {high}")
        values[name] = value
    frequency = _number("frequency_penalty", given.get("frequency_penalty", 0.0))
    repetition = _number("repetition_penalty", given.get("repetition_penalty", 1.0))
    if not BOUNDS["frequency_penalty"][0] <= frequency <= BOUNDS["frequency_penalty"][1]:
        raise ValueError("frequency_penalty must be a number from -2 to 2")
    if not 0.0 < repetition <= BOUNDS["repetition_penalty"][1]:
        raise ValueError("repetition_penalty must be a number above 0, up to 2")
    return Sampling(float(values["temperature"]), int(values["top_k"]), float(values["top_p"]), float(values["min_p"]),
                    float(values["presence_penalty"])), float(frequency), float(repetition)  # fmt: skip


def options_row(sampling, frequency_penalty: float = 0.0, repetition_penalty: float = 1.0) -> tuple[list[float], list[float]]:
    """A request's sampling settings as the two rows the sampler reads: options
    (temperature, top_k, top_p, min_p, presence_penalty), as `Sampling.values()` lays them out
    (leat/sampler.py:17-25, used at leat/engine.py:569), and penalties (repetition, presence,
    frequency), which also carries the two penalties leat's server refuses today
    (leat/server.py:84-115).  Values outside the ranges leat's server and defaults allow
    (`BOUNDS`) raise ValueError: the kernels themselves check nothing, as leat's sampler does not."""
    sampling, frequency_penalty, repetition_penalty = sampling_from_request(
        {"temperature": sampling.temperature, "top_k": sampling.top_k, "top_p": sampling.top_p, "min_p": sampling.min_p,
         "presence_penalty": sampling.presence_penalty, "frequency_penalty": frequency_penalty,
         "repetition_penalty": repetition_penalty})  # fmt: skip
    options = [float(v) for v in sampling.values()]
    return options, [float(repetition_penalty), float(sampling.presence_penalty), float(frequency_penalty)]
