"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations (host NumPy arrays; nothing here touches a GPU).  They stand in for real model
logits: the sampler's cost depends on shapes and on how peaked the rows are, not on what produced
them.  Generator: numpy PCG64 seeded with 20260000 + configuration number."""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

F32 = np.float32


@dataclass
class Workload:
    name: str
    logits: np.ndarray  # (B, V) float32
    options: np.ndarray  # (B, 5) float32: temperature, top_k, top_p, min_p, presence
    penalties: np.ndarray | None  # (B, 3) float32: repetition, presence, frequency
    history: np.ndarray | None  # (B, H) int32
    uniform: np.ndarray  # (B,) float32
    seed: np.ndarray  # (B,) uint32, for the hashed draw
    position: np.ndarray  # (B,) int32
    drafted: np.ndarray | None = None  # config 4: (n, drafts) int32
    meta: dict = field(default_factory=dict)

    @property
    def rows(self) -> int:
        return self.logits.shape[0]

    @property
    def vocab(self) -> int:
        return self.logits.shape[1]

    @property
    def logit_bytes(self) -> int:
        return self.logits.size * 4


SHAPES = {1: (1, 128256), 2: (16, 151936), 3: (256, 262144), 4: (72, 151936), 5: (512, 201088)}


def _rng(config: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(20260000 + config))


def _normal(rng, rows, vocab, sigma):
    out = np.empty((rows, vocab), F32)
    for b in range(rows):  # row by row keeps the peak host memory at one row of float64
        out[b] = rng.standard_normal(vocab, dtype=F32) * F32(sigma)
    return out


def _common(rng, rows):
    uniform = rng.random(rows, dtype=F32)
    seed = rng.integers(0, 2**32, rows, dtype=np.uint64).astype(np.uint32)
    position = rng.integers(1, 4096, rows).astype(np.int32)
    return uniform, seed, position


def config1(rows: int | None = None, vocab: int | None = None) -> Workload:
    """Single-row sample: V = 128256, N(0, 3^2); T 0.8, top-k 40, top-p 0.95, repetition 1.1 over
    64 uniform history ids."""
    rng = _rng(1)
    rows, vocab = rows or SHAPES[1][0], vocab or SHAPES[1][1]
    logits = _normal(rng, rows, vocab, 3.0)
    options = np.tile(np.array([0.8, 40, 0.95, 0.0, 0.0], F32), (rows, 1))
    penalties = np.tile(np.array([1.1, 0.0, 0.0], F32), (rows, 1))
    history = rng.integers(0, vocab, (rows, 64)).astype(np.int32)
    return Workload("c1_single_row", logits, options, penalties, history, *_common(rng, rows))


def config2(rows: int | None = None, vocab: int | None = None) -> Workload:
    """Batched server decode step: B = 16, V = 151936, N(0, 2^2) plus 5 spikes of +12 per row;
    per-row T in [0.5, 1.2], top-k 64, min-p 0.05, presence 0.3, frequency 0.2, repetition 1.05 over
    a 1024-token Zipf(1.1) history."""
    rng = _rng(2)
    rows, vocab = rows or SHAPES[2][0], vocab or SHAPES[2][1]
    logits = _normal(rng, rows, vocab, 2.0)
    for b in range(rows):
        logits[b, rng.choice(vocab, 5, replace=False)] = F32(12.0)
    options = np.zeros((rows, 5), F32)
    options[:, 0] = rng.uniform(0.5, 1.2, rows).astype(F32)
    options[:, 1], options[:, 2], options[:, 3] = 64, 1.0, 0.05
    penalties = np.tile(np.array([1.05, 0.3, 0.2], F32), (rows, 1))
    by_rank = rng.permutation(vocab)
    ranks = np.minimum(rng.zipf(1.1, (rows, 1024)), vocab) - 1
    history = by_rank[ranks].astype(np.int32)
    return Workload("c2_server_step", logits, options, penalties, history, *_common(rng, rows))


def config3(rows: int | None = None, vocab: int | None = None) -> Workload:
    """Large batch, large vocabulary: B = 256, V = 262144, N(0, 4^2) with 1 % of entries raised by
    U(5, 15); T 1, top-k 256, top-p 0.9, repetition 1.1 over 2048 uniform history ids; a quarter
    of the rows greedy."""
    rng = _rng(3)
    rows, vocab = rows or SHAPES[3][0], vocab or SHAPES[3][1]
    logits = _normal(rng, rows, vocab, 4.0)
    for b in range(rows):
        at = rng.choice(vocab, max(vocab // 100, 1), replace=False)
        logits[b, at] += rng.uniform(5.0, 15.0, len(at)).astype(F32)
    options = np.tile(np.array([1.0, 256, 0.9, 0.0, 0.0], F32), (rows, 1))
    options[rng.permutation(rows)[: rows // 4], 0] = 0.0
    penalties = np.tile(np.array([1.1, 0.0, 0.0], F32), (rows, 1))
    history = rng.integers(0, vocab, (rows, 2048)).astype(np.int32)
    return Workload("c3_large_batch", logits, options, penalties, history, *_common(rng, rows))


def config4(sequences: int | None = None, vocab: int | None = None, drafts: int = 8) -> Workload:
    """Speculative verification: 8 sequences x (8 drafts + 1 bonus) rows, V = 151936, N(0, 3^2),
    each draft's logit raised by 6 with probability 0.7; top-k 40, top-p 0.95, T 1."""
    rng = _rng(4)
    n, vocab = sequences or 8, vocab or SHAPES[4][1]
    ran = drafts + 1
    logits = _normal(rng, n * ran, vocab, 3.0)
    drafted = rng.integers(0, vocab, (n, drafts)).astype(np.int32)
    boosted = rng.random((n, drafts)) < 0.7
    for i in range(n):
        for j in range(drafts):
            if boosted[i, j]:
                logits[i * ran + j, drafted[i, j]] += F32(6.0)
    options = np.tile(np.array([1.0, 40, 0.95, 0.0, 0.0], F32), (n * ran, 1))
    w = Workload("c4_draft_verify", logits, options, None, None, *_common(rng, n * ran), drafted=drafted)
    w.meta = {"sequences": n, "drafts": drafts}
    return w


def config5(rows: int | None = None, vocab: int | None = None) -> Workload:
    """Vocabulary-sharded sampling: B = 512, V = 201088, N(0, 3^2); T 0.7, top-k 64, top-p 0.95,
    repetition 1.1 over 512 uniform history ids (replicated on every rank)."""
    rng = _rng(5)
    rows, vocab = rows or SHAPES[5][0], vocab or SHAPES[5][1]
    logits = _normal(rng, rows, vocab, 3.0)
    options = np.tile(np.array([0.7, 64, 0.95, 0.0, 0.0], F32), (rows, 1))
    penalties = np.tile(np.array([1.1, 0.0, 0.0], F32), (rows, 1))
    history = rng.integers(0, vocab, (rows, 512)).astype(np.int32)
    return Workload("c5_vocab_sharded", logits, options, penalties, history, *_common(rng, rows))


CONFIGS = {1: config1, 2: config2, 3: config3, 4: config4, 5: config5}


def shard_bounds(vocab: int, parts: int, part: int) -> tuple[int, int]:
    """Contiguous vocabulary slices, a tensor-parallel lm_head's layout: rank r owns
    [r * ceil4(V / N), ...) with slice widths rounded up to a multiple of 4 floats (16 bytes)."""
    width = -(-vocab // parts)
    width = -(-width // 4) * 4
    start = min(part * width, vocab)
    return start, min(start + width, vocab)
