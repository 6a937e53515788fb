"""The accept step of speculative decoding on the device: what the host loop of
leat/engine.py:612-626 computes from a speculative step's drafts and draws."""

from __future__ import annotations

import torch

from leat_b200 import _lib


def verify_draft(drafted: torch.Tensor, sampled: torch.Tensor, greedy: torch.Tensor | None = None
                 ) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
    """drafted (n, drafts) and sampled (n, drafts + 1) int32 -> accepted (n,) and tokens
    (n, drafts + 1) int32 padded with -1.  A draft is kept while it equals what the target sampled
    at its position (leat/engine.py:614-616); the tokens are sampled[0..accepted].  With `greedy`
    (n, drafts + 1), the variant: a draft is kept while it equals the target's greedy token, and
    the tokens are the kept drafts then the token sampled after them."""
    if drafted.dtype != torch.int32 or sampled.dtype != torch.int32 or not sampled.is_cuda:
        raise ValueError("drafted and sampled must be int32 CUDA tensors")
    n, ran = sampled.shape
    if tuple(drafted.shape) != (n, ran - 1):
        raise ValueError("drafted must be (n, drafts) and sampled (n, drafts + 1)")
    drafted, sampled = drafted.contiguous(), sampled.contiguous()
    if greedy is not None:
        if tuple(greedy.shape) != (n, ran) or greedy.dtype != torch.int32:
            raise ValueError("greedy must be (n, drafts + 1) int32")
        greedy = greedy.contiguous()
    accepted = torch.empty(n, dtype=torch.int32, device=sampled.device)
    tokens = torch.empty((n, ran), dtype=torch.int32, device=sampled.device)
    with torch.cuda.device(sampled.device):
        _lib.check(_lib.lib.leat_verify_draft(
            drafted.data_ptr(), sampled.data_ptr(), None if greedy is None else greedy.data_ptr(), n, ran - 1,
            accepted.data_ptr(), tokens.data_ptr(), torch.cuda.current_stream().cuda_stream), "leat_verify_draft")  # fmt: skip
    return accepted, tokens


def settle_draft(history, slots: torch.Tensor, last: torch.Tensor, drafted: torch.Tensor, sampled: torch.Tensor,
                 accepted: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """What follows the accept step, on the device too (leat/engine.py:609-631 and `_settled`,
    :677-686): `history` (a leat_b200.history.SlotHistory on the GPU) takes, for sequence i in slot
    slots[i], the tokens that were run up to its kept row, last[i] then drafted[i, :accepted[i]],
    markup left out, as leat's `_seen_rows[row]` holds them.  Returns next (n,), the token each
    sequence runs in the next step (sampled[i, accepted[i]]), and row (n,), the row whose hidden
    state its slot keeps (i * (drafts + 1) + accepted[i]).  No host synchronisation: the next step's
    inputs are device tensors, as a decode step's are (leat/engine.py:564-566)."""
    n, ran = sampled.shape
    d = sampled.device
    if not sampled.is_cuda or history.ids.device != d:
        raise ValueError("sampled and the history must be on the same CUDA device")
    as32 = lambda x: x.to(device=d, dtype=torch.int32).contiguous()  # noqa: E731
    slots, last, drafted, sampled, accepted = as32(slots), as32(last), as32(drafted), as32(sampled), as32(accepted)
    if tuple(drafted.shape) != (n, ran - 1) or slots.numel() != n or last.numel() != n or accepted.numel() != n:
        raise ValueError("drafted must be (n, drafts); slots, last and accepted (n,)")
    text = history.text.view(torch.uint8)
    nxt = torch.empty(n, dtype=torch.int32, device=d)
    row = torch.empty(n, dtype=torch.int32, device=d)
    with torch.cuda.device(d):
        _lib.check(_lib.lib.leat_settle_draft(
            accepted.data_ptr(), last.data_ptr(), drafted.data_ptr() if ran > 1 else None, sampled.data_ptr(),
            slots.data_ptr(), n, ran - 1, history.ids.data_ptr(), history.count.data_ptr(), history.capacity,
            text.data_ptr(), history.vocab, nxt.data_ptr(), row.data_ptr(),
            torch.cuda.current_stream().cuda_stream), "leat_settle_draft")  # fmt: skip
    return nxt, row
