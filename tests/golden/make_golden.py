"""Writes tests/golden/config<N>.npz: the CPU oracle's answers for the five benchmark configurations
at full size, so that an edit of the oracle cannot move the target unnoticed and the GPU tests can
check every row without running the oracle.

    python tests/golden/make_golden.py [config numbers]

Per configuration and draw mode (U: supplied uniforms, G: hashed Gumbel-max), for every row: the
sampled id, the greedy id, the number of survivors, the cut, the first eight survivor ids (likeliest
first, -1 padded) and the oracle's margin (rows with a margin under 1e-5 are nucleus-boundary ties,
which the tests exempt).  Inputs come from leat_b200/workloads.py (numpy PCG64, seed 20260000 + N);
sums in the CUDA path's block order."""

from __future__ import annotations

import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

FIRST = 8


def answers(w, mode: str, rows=None) -> dict:
    from oracle import sampler_oracle as oracle

    rows = range(w.rows) if rows is None else rows

    def one(b: int):
        sel = slice(b, b + 1)
        r = oracle.sample(w.logits[sel], w.options[sel], w.seed[sel], w.position[sel],
                          history=None if w.history is None else w.history[sel],
                          penalties=None if w.penalties is None else w.penalties[sel],
                          uniform_draws=w.uniform[sel] if mode == "U" else None, order="block")  # fmt: skip
        first = np.full(FIRST, -1, np.int32)
        if r.kept[0] > 0 and w.options[b, 0] > 0:
            n = min(FIRST, len(r.prob_ids[0]))
            first[:n] = r.prob_ids[0][:n]
        return r.ids[0, 0], r.greedy[0], r.kept[0], r.cut[0], r.margin[0], first

    with ThreadPoolExecutor(8) as pool:
        got = list(pool.map(one, rows))
    ids, greedy, kept, cut, margin, first = (np.array(x) for x in zip(*got))
    return {f"{mode}_ids": ids.astype(np.int32), f"{mode}_greedy": greedy.astype(np.int32), f"{mode}_kept": kept.astype(np.int32),
            f"{mode}_cut": cut.astype(np.float32), f"{mode}_margin": margin.astype(np.float64), f"{mode}_first": first.astype(np.int32)}  # fmt: skip


def main() -> None:
    from leat_b200 import workloads

    for config in [int(x) for x in sys.argv[1:]] or [1, 2, 3, 4, 5]:
        w = workloads.CONFIGS[config]()
        out = {"rows": np.int32(w.rows), "vocab": np.int32(w.vocab)}
        for mode in ("U", "G"):
            out.update(answers(w, mode))
        np.savez_compressed(Path(__file__).resolve().parent / f"config{config}.npz", **out)
        print(f"config {config}: {w.rows} rows x {w.vocab}", flush=True)


if __name__ == "__main__":
    main()
