"""The two ops of leat/ops.py that the sampler is made of, over the CUDA library: argmax
(leat/ops.py:496-500) and cutoff (leat/ops.py:503-515, with the exact cut of :518-529)."""

from __future__ import annotations

import torch

from leat_b200.sampler import default_sampler


def argmax(x: torch.Tensor) -> torch.Tensor:
    """Index of each row's largest value, the first on ties: (B, V) float32 -> (B, 1) int32."""
    return default_sampler(x.shape[0], x.shape[1], x.device).argmax(x)


def cutoff(scores: torch.Tensor, top_k, top_p, min_p) -> torch.Tensor:
    """The score below which each row of scores (B, V) drops its tokens, each option (B, 1):
    -inf where no option is set."""
    return default_sampler(scores.shape[0], scores.shape[1], scores.device).cutoff(scores, top_k, top_p, min_p)
