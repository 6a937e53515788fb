"""CPU oracle for leat's token sampler: TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

A NumPy restatement, in float32, of the exact reference sampler (the one leat takes with
LEAT_KERNELS=ref): leat/sampler.py:31-73 (sample, _uniform, _hash), leat/ops.py:496-529 (argmax,
cutoff, _cutoff) and the host accept loop of leat/engine.py:609-626.  Only tests, the smoke check
and the CPU-baseline legs of the benchmark may import it; the shipped package never does.

Parity pin.  The reference needs tinygrad (a git dependency that is not vendored), which is absent
where this was written, so the reference itself could not be run.  The restatement is pinned
instead against every known answer the reference's own tests hold for this path
(tests/test_sampler.py:37-93, tests/test_kernels.py:927-955, tests/helpers.py:354-361); those pin
greedy ids, kept sets, determinism, row independence and distributions.  They do not pin the last
bits of exp/log/cumsum, so float behaviour below that level is PARITY UNPINNED and is fixed here by
stated conventions:

* x / T is evaluated as x * (1 / max(T, 1e-6)) (`scale="reciprocal"`), as the reference's authors
  say tinygrad does (leat/kernels/common.py:166-168); `scale="divide"` gives the IEEE quotient.
* exp(x) = exp2(x * log2(e)) and log(x) = log2(x) * ln(2), tinygrad's own lowering.
* cumsum/sum order: `order="sequential"` is the plain left-to-right float32 running sum;
  `order="block"` is the order of the CUDA path's block scan (a 32-wide Kogge-Stone scan per
  segment of 32 ranks, segment totals added left to right).  The two differ only in last bits, and
  so only at nucleus-boundary ties, which `Result.margin` exposes.

Extensions with no reference behaviour (conventions, stated in the functions below): the
supplied-uniform inverse-CDF draw, repetition and frequency penalties from history counts,
post-filter probabilities, greedy-match draft verification, vocabulary shards.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

F32 = np.float32
LOG2E = F32(1.0 / math.log(2.0))
LN2 = F32(math.log(2.0))
T_FLOOR = F32(1e-6)
NEG_INF = F32(-np.inf)


# ----------------------------------------------------------------------------------------------
# elementary functions, as tinygrad lowers them
# ----------------------------------------------------------------------------------------------


def exp32(x):
    """exp(x) as exp2(x * log2 e), float32 (leat/ops.py:524 through tinygrad's Tensor.exp)."""
    return np.exp2(np.asarray(x, F32) * LOG2E).astype(F32)


def log32(x):
    """log(x) as log2(x) * ln 2, float32; log(0) = -inf (leat/ops.py:514)."""
    with np.errstate(divide="ignore", invalid="ignore"):
        return (np.log2(np.asarray(x, F32)) * LN2).astype(F32)


def lowbias32(x):
    """leat/sampler.py:67-73: lowbias32 with every product wrapped to 32 bits."""
    x = np.atleast_1d(np.asarray(x)).astype(np.uint32)
    with np.errstate(over="ignore"):
        x = (x ^ (x >> np.uint32(16))) * np.uint32(0x7FEB352D)
        x = (x ^ (x >> np.uint32(15))) * np.uint32(0x846CA68B)
        return x ^ (x >> np.uint32(16))


def row_keys(seed, position):
    """leat/sampler.py:62: key = h(h(seed) + u32(position)), one per row."""
    seed = np.atleast_1d(np.asarray(seed)).astype(np.uint32)
    position = np.atleast_1d(np.asarray(position)).astype(np.int64).astype(np.uint32)
    with np.errstate(over="ignore"):
        return lowbias32(lowbias32(seed) + position)


def uniform(seed, position, vocab: int, start: int = 0):
    """leat/sampler.py:58-64: (rows, vocab) float32 in (0, 1), hashed from seed, position and the
    token's index; `start` offsets the index for a vocabulary shard."""
    key = row_keys(seed, position).reshape(-1, 1)
    index = (np.arange(vocab, dtype=np.int64) + start).astype(np.uint32).reshape(1, -1)
    bits = lowbias32(index ^ key)
    return ((bits >> np.uint32(9)).astype(F32) + F32(0.5)) * F32(2.0**-23)


def gumbel(u):
    """leat/sampler.py:53: -log(-log(u))."""
    return -log32(-log32(u))


def argmax(x):
    """leat/ops.py:496-500: index of each row's largest value, the first on ties: (B, 1) int32."""
    x = np.asarray(x, F32)
    return np.argmax(x, axis=-1).astype(np.int32).reshape(-1, 1)


# ----------------------------------------------------------------------------------------------
# running sums
# ----------------------------------------------------------------------------------------------


def running_sum(w, order: str = "sequential"):
    """Inclusive float32 running sum of a 1-D array in the stated order."""
    w = np.asarray(w, F32)
    if order == "sequential":
        return np.cumsum(w, dtype=F32)
    if order != "block":
        raise ValueError(order)
    n = len(w)
    if n == 0:
        return w.copy()
    segments = -(-n // 32)
    x = np.zeros(segments * 32, F32)
    x[:n] = w
    x = x.reshape(segments, 32)
    for d in (1, 2, 4, 8, 16):  # Kogge-Stone: every lane adds the value d lanes to its left
        x[:, d:] = x[:, d:] + x[:, :-d]
    offsets = np.zeros(segments, F32)
    for i in range(1, segments):
        offsets[i] = offsets[i - 1] + x[i - 1, 31]
    return (offsets.reshape(-1, 1) + x).reshape(-1)[:n].astype(F32)


# ----------------------------------------------------------------------------------------------
# penalties and temperature
# ----------------------------------------------------------------------------------------------


def history_counts(history, history_len, vocab: int, start: int = 0):
    """Per-row count of each token id in the row's history (B, H) int32, of which the first
    history_len[b] entries count; ids outside [start, start + vocab) are ignored.  Extension: the
    reference keeps a bool mask instead (leat/engine.py:768-781); count > 0 is that mask."""
    history = np.asarray(history, np.int64)
    rows = history.shape[0]
    history_len = np.full(rows, history.shape[1]) if history_len is None else np.asarray(history_len)
    counts = np.zeros((rows, vocab), np.int32)
    for b in range(rows):
        ids = history[b, : int(history_len[b])] - start
        ids = ids[(ids >= 0) & (ids < vocab)]
        np.add.at(counts[b], ids, 1)
    return counts


def penalise(logits, counts, repetition, presence, frequency):
    """One row.  Where count > 0: repetition first (l > 0 ? l / r : l * r), then
    l -= presence + frequency * count (the product and the sum each rounded to float32).  With
    r = 1 and frequency = 0 this is leat/sampler.py:48-49 exactly; repetition and frequency are
    extensions with no reference behaviour."""
    l = np.asarray(logits, F32)
    if counts is None:
        return l
    hit = np.asarray(counts) > 0
    r, p, f = F32(repetition), F32(presence), F32(frequency)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        rep = np.where(l > 0, l / r, l * r).astype(F32)
        off = (p + (f * np.asarray(counts).astype(F32)).astype(F32)).astype(F32)
        return np.where(hit, (rep - off).astype(F32), l).astype(F32)


def soft_cap(logits, cap):
    """leat/model.py:419-423: logits = tanh(logits / cap) * cap, the soft cap a model puts on its
    logits before they are sampled (cap 0 or None: none).  The reference evaluates it in float32
    through tinygrad, which cannot be run here (PARITY UNPINNED); the convention fixed here and in the
    CUDA path is double precision rounded once to float32, which both sides reproduce exactly."""
    l = np.asarray(logits, F32)
    if not cap:
        return l
    with np.errstate(invalid="ignore", over="ignore"):
        return (np.tanh(l.astype(np.float64) / np.float64(F32(cap))) * np.float64(F32(cap))).astype(F32)


def scale_scores(l, temperature, scale: str = "reciprocal"):
    """leat/sampler.py:50: scores = logits / max(T, 1e-6)."""
    t = np.maximum(F32(temperature), T_FLOOR)
    with np.errstate(invalid="ignore", over="ignore"):
        if scale == "reciprocal":
            return (np.asarray(l, F32) * (F32(1.0) / t)).astype(F32) + F32(0.0)
        if scale == "divide":
            return (np.asarray(l, F32) / t).astype(F32) + F32(0.0)
    raise ValueError(scale)


# ----------------------------------------------------------------------------------------------
# the cut (leat/ops.py:503-529)
# ----------------------------------------------------------------------------------------------


@dataclass
class Cut:
    top: np.float32
    by_k: np.float32
    by_p: np.float32
    cut: np.float32
    margin: float  # smallest relative distance of a top-p comparison from flipping


def cutoff_row(ranked, top_k, top_p, min_p, order: str = "sequential") -> Cut:
    """leat/ops.py:518-529 then :514-515 for one row whose scores are already sorted descending."""
    ranked = np.asarray(ranked, F32)
    n = len(ranked)
    top_k, top_p, min_p = F32(top_k), F32(top_p), F32(min_p)
    k = top_k if top_k > 0 else F32(n)
    in_k = int(min(math.floor(float(k)), n))  # ranks 1..in_k are those with rank <= k
    with np.errstate(invalid="ignore", over="ignore"):
        weights = exp32(ranked[:in_k] - ranked[0])
    incl = running_sum(weights, order)
    likelier = (incl - weights).astype(F32)
    kept = incl[-1] if in_k else F32(0.0)
    by_k = ranked[in_k - 1]
    bound = F32(top_p * kept)
    keep = likelier < bound
    keep[0] = True
    by_p = ranked[:in_k][keep].min()
    with np.errstate(invalid="ignore"):
        margin = float(np.min(np.abs(likelier[1:] - bound)) / kept) if (top_p < 1 and in_k > 1) else 1.0
        cut = np.maximum(by_p if top_p < 1 else by_k, (ranked[0] + log32(min_p)).astype(F32))
    if not (top_k > 0 or top_p < 1 or min_p > 0):
        cut = NEG_INF
    return Cut(ranked[0], by_k, by_p, F32(cut), margin)


def cutoff(scores, top_k, top_p, min_p, order: str = "sequential"):
    """leat/ops.py:503-515: (B, V) scores and (B, 1) options -> (B, 1) cut."""
    scores = np.asarray(scores, F32)
    rows = scores.shape[0]
    opts = [np.broadcast_to(np.asarray(o, F32).reshape(-1), (rows,)) for o in (top_k, top_p, min_p)]
    out = np.empty((rows, 1), F32)
    for b in range(rows):
        ranked = -np.sort(-scores[b])
        out[b, 0] = cutoff_row(ranked, opts[0][b], opts[1][b], opts[2][b], order).cut
    return out


def cuts_f64(scores, top_k, top_p):
    """An independent float64 statement of the three cuts for one row, after the reference's own
    cross-check (tests/helpers.py:354-361): the top score, the k-th (the last at k = 0), and the
    last of those whose likelier ones' share of the top k's mass falls short of top_p."""
    ranked = np.sort(np.asarray(scores, np.float64))[::-1]
    ranked = ranked[: int(top_k) or len(ranked)]
    w = np.exp(ranked - ranked[0])
    before = np.cumsum(w) - w
    last = max(int((before < top_p * w.sum()).sum()), 1) - 1
    return ranked[0], ranked[-1], ranked[last]


# ----------------------------------------------------------------------------------------------
# sample()
# ----------------------------------------------------------------------------------------------


@dataclass
class Result:
    ids: np.ndarray  # (B, 1) int32: the sampled token per row (leat/sampler.py:55)
    greedy: np.ndarray  # (B,) int32: argmax of the penalised logits
    cut: np.ndarray  # (B,) float32
    kept: np.ndarray  # (B,) int32: number of survivors (scores >= cut)
    prob_ids: list = field(default_factory=list)  # per row: survivor ids, likeliest first
    probs: list = field(default_factory=list)  # per row: their probabilities
    margin: np.ndarray | None = None  # (B,) smallest relative distance of a decision from flipping
    penalised: np.ndarray | None = None  # (B, V) penalised logits, when asked for
    notes: dict = field(default_factory=dict)  # row -> nucleus_boundary() of a row whose margin is under 1e-5


def _rows(x, rows, width=None, dtype=None):
    x = np.asarray(x) if dtype is None else np.asarray(x, dtype)
    if width is None:
        return np.broadcast_to(x.reshape(-1), (rows,))
    return np.broadcast_to(x.reshape(-1, width), (rows, width))


def sample(
    logits, options, seed=None, position=0, seen=None, *,
    history=None, history_len=None, penalties=None, uniform_draws=None,
    scale: str = "reciprocal", order: str = "sequential", survivors: bool = True,
    keep_penalised: bool = False, vocab_start: int = 0, softcap: float = 0.0,
) -> Result:  # fmt: skip
    """leat/sampler.py:31-55 for float32 `logits` (B, V) and `options` (B|1, 5) rows of
    [temperature, top_k, top_p, min_p, presence_penalty].

    Reference modes: `seen` (B, V) bool marks the tokens presence_penalty lowers; the draw is
    Gumbel-max over uniforms hashed from `seed` (B|1) uint32 and `position` (scalar or (B,)).

    Extensions: `history` (B, H) int32 with `history_len` (B,) gives per-token counts (a `seen`
    mask counts as one occurrence where the history has none); `penalties` (B|1, 3) rows of
    [repetition, presence, frequency] replace the options' presence column; `softcap` applies the
    model's soft cap (soft_cap) to the logits first; `uniform_draws` (B,)
    switches the draw to inverse-CDF: survivors ordered by descending score, ties by ascending id,
    weights exp(score - top), the first survivor whose running weight exceeds u * total, else the
    last.  `vocab_start` offsets the hashed index (a vocabulary shard)."""
    logits = soft_cap(np.asarray(logits, F32), softcap)  # (the model's own last step, before any penalty)
    rows, vocab = logits.shape
    options = _rows(options, rows, 5, F32)
    counts = None
    if history is not None:
        counts = history_counts(history, history_len, vocab)
    if seen is not None:
        mask = np.asarray(seen).astype(bool).astype(np.int32)
        counts = mask if counts is None else np.maximum(counts, mask)
    if penalties is None:
        penalties = np.stack([np.ones(rows, F32), options[:, 4], np.zeros(rows, F32)], axis=1)
    penalties = _rows(penalties, rows, 3, F32)
    if uniform_draws is None:
        keys = np.broadcast_to(row_keys(seed, position), (rows,))
    else:
        uniform_draws = _rows(uniform_draws, rows, None, F32)

    out = Result(np.zeros((rows, 1), np.int32), np.zeros(rows, np.int32), np.zeros(rows, F32),
                 np.zeros(rows, np.int32), margin=np.ones(rows))  # fmt: skip
    if keep_penalised:
        out.penalised = np.empty_like(logits)
    index = (np.arange(vocab, dtype=np.int64) + vocab_start).astype(np.uint32)
    for b in range(rows):
        temperature, top_k, top_p, min_p, _ = options[b]
        l = penalise(logits[b], None if counts is None else counts[b], *penalties[b])
        if keep_penalised:
            out.penalised[b] = l
        out.greedy[b] = int(np.argmax(l))
        s = scale_scores(l, temperature, scale)
        by_rank = np.argsort(-s, kind="stable")  # descending score, ties by ascending id
        ranked = s[by_rank]
        c = cutoff_row(ranked, top_k, top_p, min_p, order)
        margin = c.margin
        live = int(np.count_nonzero(s >= c.cut))
        out.cut[b], out.kept[b] = c.cut, live
        if survivors or uniform_draws is not None:
            with np.errstate(invalid="ignore", over="ignore"):
                w = exp32(ranked[:live] - ranked[0])
            incl = running_sum(w, order)
            total = incl[-1]
            out.prob_ids.append((by_rank[:live] + vocab_start).astype(np.int32))
            out.probs.append((w / total).astype(F32))
        if not temperature > 0:
            out.ids[b, 0] = out.greedy[b] + vocab_start
        elif uniform_draws is None:
            bits = lowbias32(index ^ keys[b])
            u = ((bits >> np.uint32(9)).astype(F32) + F32(0.5)) * F32(2.0**-23)
            with np.errstate(invalid="ignore"):
                drawn = np.where(s >= c.cut, (s + gumbel(u)).astype(F32), NEG_INF)
            first = int(np.argmax(drawn))
            out.ids[b, 0] = first + vocab_start
            if live > 1:
                two = np.partition(drawn, vocab - 2)[-2:]
                margin = min(margin, float((two[1] - two[0]) / max(abs(float(two[1])), 1.0)))
        else:
            bound = F32(uniform_draws[b] * total)
            over = np.nonzero(incl > bound)[0]
            j = int(over[0]) if len(over) else live - 1
            out.ids[b, 0] = int(by_rank[j]) + vocab_start
            margin = min(margin, float(np.min(np.abs(incl - bound)) / total))
        out.margin[b] = margin
        if margin < 1e-5 and temperature > 0:
            out.notes[b] = nucleus_boundary(s, top_k, top_p)
    return out


# ----------------------------------------------------------------------------------------------
# draft verification (leat/engine.py:609-626)
# ----------------------------------------------------------------------------------------------


def verify_draft(drafted, sampled):
    """The reference's accept loop: per sequence, kept = the first j with drafted[j] != sampled[j],
    else the number of drafts; the tokens emitted are sampled[0..kept].  drafted (n, d) and
    sampled (n, d + 1) int32 -> kept (n,), tokens (n, d + 1) padded with -1."""
    drafted, sampled = np.asarray(drafted, np.int32), np.asarray(sampled, np.int32)
    n, d = drafted.shape
    kept = np.full(n, d, np.int32)
    tokens = np.full((n, d + 1), -1, np.int32)
    for i in range(n):
        for j in range(d):
            if drafted[i, j] != sampled[i, j]:
                kept[i] = j
                break
        tokens[i, : kept[i] + 1] = sampled[i, : kept[i] + 1]
    return kept, tokens


def verify_draft_greedy(drafted, greedy, sampled):
    """Variant (an extension): a draft is accepted while it equals the target's greedy token at its
    position; the token after the accepted prefix is the one sampled at that position.  Tokens
    emitted: drafted[0..kept) then sampled[kept]."""
    drafted, greedy = np.asarray(drafted, np.int32), np.asarray(greedy, np.int32)
    sampled = np.asarray(sampled, np.int32)
    n, d = drafted.shape
    kept = np.full(n, d, np.int32)
    tokens = np.full((n, d + 1), -1, np.int32)
    for i in range(n):
        for j in range(d):
            if drafted[i, j] != greedy[i, j]:
                kept[i] = j
                break
        tokens[i, : kept[i]] = drafted[i, : kept[i]]
        tokens[i, kept[i]] = sampled[i, kept[i]]
    return kept, tokens


def settle_draft(ids, count, capacity, text, slots, last, drafted, sampled, accepted):
    """What leat does after the accept loop (leat/engine.py:609-631, `_settled` :677-686), with each
    slot's generated tokens kept as a ring of ids (ids (slots, capacity), count (slots,)) instead of
    the dense `_seen` mask: the slot takes the tokens that were run up to the kept row, last[i] then
    drafted[i, :accepted[i]], except markup (`text[token]` false); next[i] = sampled[i, accepted[i]];
    row[i] = i * (drafts + 1) + accepted[i].  Updates ids and count in place."""
    n, ran = np.asarray(sampled).shape
    nxt, row = np.zeros(n, np.int32), np.zeros(n, np.int32)
    for i in range(n):
        kept = int(accepted[i])
        for token in [int(last[i]), *[int(t) for t in drafted[i][:kept]]]:
            if 0 <= token < len(text) and text[token]:
                ids[slots[i], count[slots[i]] % capacity] = token
                count[slots[i]] += 1
        nxt[i], row[i] = sampled[i][kept], i * ran + kept
    return nxt, row


def nucleus_boundary(scores, top_k, top_p):
    """For a row whose draw hangs on a top-p comparison: the rank at which the likelier mass comes
    closest to top_p * kept, with that mass and that bound in both summation orders, for the log of
    rows exempted as nucleus-boundary ties."""
    ranked = -np.sort(-np.asarray(scores, F32))
    n = len(ranked)
    in_k = int(min(math.floor(float(top_k)) if top_k > 0 else n, n))
    with np.errstate(invalid="ignore", over="ignore"):
        weights = exp32(ranked[:in_k] - ranked[0])
    out = {}
    for order in ("sequential", "block"):
        incl = running_sum(weights, order)
        likelier = (incl - weights).astype(F32)
        bound = F32(F32(top_p) * incl[-1])
        j = int(np.argmin(np.abs(likelier[1:] - bound))) + 1 if in_k > 1 else 0
        out[order] = {"rank": j, "likelier": float(likelier[j]), "top_p_times_kept": float(bound)}
    return out


# ----------------------------------------------------------------------------------------------
# vocabulary shards: what each rank contributes, for host-side tests of the gather
# ----------------------------------------------------------------------------------------------


def local_candidates(logits_slice, options, start, cap, *, history=None, history_len=None,
                     penalties=None, seen=None, scale: str = "reciprocal"):  # fmt: skip
    """What one vocabulary shard owning ids [start, start + width) hands to the gather: per row,
    every (score, global id) of its slice whose score is at least the slice's k-th largest
    (k = top_k, or the whole slice when top_k = 0), likeliest first, ties by ascending id; rows
    longer than `cap` are reported by their true count so the caller can tell.  Greedy rows
    (temperature 0) contribute their penalised logits' best instead.  Returns counts (B,),
    values (B, cap) float32 padded with -inf, ids (B, cap) int32 padded with -1, and the greedy
    (value, id) per row."""
    logits_slice = np.asarray(logits_slice, F32)
    rows, width = logits_slice.shape
    options = _rows(options, rows, 5, F32)
    counts_h = None
    if history is not None:
        counts_h = history_counts(history, history_len, width, start)
    if seen is not None:
        mask = np.asarray(seen).astype(bool).astype(np.int32)
        counts_h = mask if counts_h is None else np.maximum(counts_h, mask)
    if penalties is None:
        penalties = np.stack([np.ones(rows, F32), options[:, 4], np.zeros(rows, F32)], axis=1)
    penalties = _rows(penalties, rows, 3, F32)
    count = np.zeros(rows, np.int32)
    values = np.full((rows, cap), NEG_INF, F32)
    ids = np.full((rows, cap), -1, np.int32)
    best = np.zeros(rows, F32)
    best_id = np.zeros(rows, np.int32)
    for b in range(rows):
        l = penalise(logits_slice[b], None if counts_h is None else counts_h[b], *penalties[b])
        best_id[b] = int(np.argmax(l)) + start
        best[b] = l[best_id[b] - start]
        s = scale_scores(l, options[b, 0], scale)
        by_rank = np.argsort(-s, kind="stable")
        k = int(options[b, 1]) if options[b, 1] > 0 else width
        kth = s[by_rank[min(k, width) - 1]]
        n = int(np.count_nonzero(s >= kth))
        count[b] = n
        m = min(n, cap)
        values[b, :m] = s[by_rank[:m]]
        ids[b, :m] = by_rank[:m] + start
    return count, values, ids, best, best_id
