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
