"""Benchmark of the sampling path: rows/s of one decode step's sampling on synthetic logits.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the sampler over one batch of logits.  Every N runs the same workload, the
largest configuration: 512 rows x 201088 tokens (temperature 0.7, top-k 64, top-p 0.95, repetition
1.1 over a 512-token history, one supplied uniform per row), whose logits (412 MB) are larger than
L2, so every step reads HBM.  N = 1 is one call of the library's leat_sample on resident inputs;
N > 1 (under torchrun, one process per GPU) splits the vocabulary into N contiguous slices, one
per rank, with one exchange of candidates per step ("strong" scaling: the work is fixed).

Exactly K steps are timed, each a replay of a captured CUDA graph, with a CUDA event after every
step on the launching stream: `ms_per_step` is the timed region divided by K, `median_ms` and
`p95_ms` come from the per-step events.  The last line printed by rank 0 is one JSON object; at
N = 1 `all_configs` in it holds the device-timed figures of every configuration.

--impl reference times the CPU restatement of leat's exact sampler (oracle/) on the host's cores
for the same workload: leat itself needs tinygrad, which is not installed here, so its own code
cannot be run.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0  # an earlier measurement on this pool, used when MEASURED_PEAKS.json is absent
NORTH_STAR_HBM_GBS = 8000.0
L2_BYTES = 126 << 20
# DRAM bytes filter_kernel moves per algorithmic byte, from one ncu capture of a launch on this very
# workload (512 rows x 201088): (dram__bytes_read.sum + dram__bytes_write.sum) / (B x V x 4)
# = (411.93 + 3.77) MB / 411.83 MB; 160 rows of the large-batch configuration gave 1.02.
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0094
HEADLINE = 5  # the configuration every N runs
CPU_SAMPLE_ROWS = 32  # rows of the headline workload the CPU arm times per step
# Steps a replayed graph holds, back to back.  In leat's engine the sampler's kernels sit inside the
# decode step's graph, after the model's; launching a graph (about 4.5 us here) is the engine's cost,
# paid once per decode step whatever the sampler does, so a graph of one sampler step would count it
# against the sampler.  (The line also carries the figure for one step per graph.)
STEPS_PER_GRAPH = 10


def steps_per_graph(steps: int) -> int:
    """The largest of 10, 5, 4, 2, 1 that divides the number of timed steps."""
    return next(s for s in (10, 5, 4, 2, 1) if steps % s == 0)

WORKLOAD_NAMES = {1: "c1_single_row", 2: "c2_server_step", 3: "c3_large_batch", 4: "c4_draft_verify", 5: "c5_vocab_sharded"}
SHAPES_ROWS = {1: 1, 2: 16, 3: 256, 4: 72, 5: 512}


def peak_hbm() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (ValueError, KeyError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


def headline_config(world: int, vocab: int) -> dict:
    """The `config` object of the JSON line: the same in both arms and at every N but for the split."""
    return {"workload": WORKLOAD_NAMES[HEADLINE], "rows": SHAPES_ROWS[HEADLINE], "vocab": vocab,
            "parallelism": f"vocab{world}", "draw": "supplied uniform"}  # fmt: skip


# ---- clocks -------------------------------------------------------------------------------------


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)  # fmt: skip
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        top = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        busy = [x for x in sm if x > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(top) if top else None,
                "reasons": reasons, "samples": len(sm)}  # fmt: skip


def keep_busy(step, ms_per_step: float, seconds: float = 0.6) -> None:
    """The timed steps last milliseconds and nvidia-smi answers every 100 ms: the same steps go on,
    untimed, for about `seconds`, so that the clocks are seen under the load that was timed.  The
    number of steps depends only on the (rank-agreed) step time, so every rank runs as many."""
    import torch

    for i in range(min(50000, int(seconds * 1e3 / max(ms_per_step, 1e-3)))):
        step(i)
    torch.cuda.synchronize()


# ---- CPU baseline (the oracle on the host's cores) ------------------------------------------------


def cpu_step_seconds(w, mode: str, pool: ThreadPoolExecutor) -> float:
    """Seconds the CPU oracle takes for one pass over the rows of `w`, one row per pool task
    (NumPy releases the GIL in its sorts)."""
    from oracle import sampler_oracle as oracle

    def one(b: int) -> int:
        sel = slice(b, b + 1)
        oracle.sample(w.logits[sel], w.options[sel], w.seed[sel], w.position[sel],
                      history=None if w.history is None else w.history[sel],
                      penalties=None if w.penalties is None else w.penalties[sel],
                      uniform_draws=w.uniform[sel] if mode == "U" else None, survivors=False)  # fmt: skip
        return 1

    start = time.perf_counter()
    sum(pool.map(one, range(w.rows)))
    return time.perf_counter() - start


def cpu_rows_per_second(w, mode: str, seconds: float, threads: int) -> tuple[float, str]:
    """Rows per second of the CPU oracle over whole passes of `w` for about `seconds`."""
    passes, spent = 0, 0.0
    with ThreadPoolExecutor(threads) as pool:
        while spent < seconds:
            spent += cpu_step_seconds(w, mode, pool)
            passes += 1
    return passes * w.rows / spent, f"{passes} passes over {w.rows} rows x {w.vocab} of {w.name} in {spent:.1f} s"


def run_reference(args) -> None:
    """The reference arm: the CPU restatement on all host threads, a step = one pass over a bounded
    sample (CPU_SAMPLE_ROWS rows) of the headline workload; rows/s does not depend on how many rows
    a pass holds (rows are independent), so the figure stands for the 512-row step."""
    from leat_b200 import workloads

    if int(os.environ.get("RANK", 0)) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", 1))
    w = workloads.CONFIGS[HEADLINE](rows=CPU_SAMPLE_ROWS)
    threads = os.cpu_count() or 1
    times = []
    with ThreadPoolExecutor(threads) as pool:
        for step in range(args.warmup + args.steps):
            seconds = cpu_step_seconds(w, "U", pool)
            if step >= args.warmup:
                times.append(seconds)
    value = w.rows / float(np.mean(times))
    sample = (f"{args.steps} steps of {w.rows} rows x {w.vocab} of {WORKLOAD_NAMES[HEADLINE]}, one row per task on "
              f"{threads} threads; ms_per_step is scaled from {w.rows} rows to {SHAPES_ROWS[HEADLINE]}")  # fmt: skip
    line = {
        "impl": "reference", "metric": "sampler rows/s", "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * SHAPES_ROWS[HEADLINE] / value,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": headline_config(world, w.vocab),
        "extrapolated_from_rows": w.rows,
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port", "sample": sample,
                         "extrapolated_from_rows": w.rows},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "leat's own sampler needs tinygrad (not installed, no network): this is the NumPy restatement of "
                "its exact path (LEAT_KERNELS=ref) on the host cores",
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ---- the GPU arm ---------------------------------------------------------------------------------


class DeviceWorkload:
    """A workload resident in HBM, its logits replicated into a pool larger than L2."""

    def __init__(self, w, device, min_pool_bytes=2 * L2_BYTES, max_copies=512, dtype=None):
        import torch

        self.w, self.device = w, device
        self.logit_bytes = w.logit_bytes if dtype is None else w.logit_bytes // 2
        copies = int(min(max_copies, max(1, -(-min_pool_bytes // self.logit_bytes))))
        if self.logit_bytes > L2_BYTES:
            copies = 1  # one buffer is already larger than L2
        base = torch.as_tensor(w.logits).to(device)
        if dtype is not None:  # the lm_head's own 16-bit output, read as it is
            base = base.to(dtype)
        self.pool = [base] + [base.clone() for _ in range(copies - 1)]
        t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
        self.options, self.penalties, self.history = t(w.options), t(w.penalties), t(w.history)
        self.uniform, self.position = t(w.uniform), t(w.position)
        self.seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
        self.out = torch.empty((w.rows, 1), dtype=torch.int32, device=device)
        self.l2_note = ("logits pool of %d buffers (%.0f MB) cycled, larger than L2" % (copies, copies * self.logit_bytes / 1e6)
                        if copies > 1 else "inputs larger than L2 (%.0f MB per step)" % (self.logit_bytes / 1e6))  # fmt: skip

    def step(self, sampler, i: int):
        return sampler.sample_full(self.pool[i % len(self.pool)], self.options, self.seed, self.position,
                                   history=self.history, penalties=self.penalties, uniform=self.uniform, out=self.out)  # fmt: skip


def capture(step, inner: int):
    """A CUDA graph holding steps 0 .. inner - 1 (launch overhead of the host taken out, as in leat's
    engine, which replays captured graphs)."""
    import torch

    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(inner):
                step(i)
    torch.cuda.synchronize()
    return graph


def timed_replays(replay, count: int) -> tuple[float, list[float]]:
    """`count` calls of replay(i) with a CUDA event after each on the current stream: milliseconds
    of the whole region, and of each call."""
    import torch

    marks = [torch.cuda.Event(enable_timing=True) for _ in range(count + 1)]
    torch.cuda.synchronize()
    marks[0].record()
    for i in range(count):
        replay(i)
        marks[i + 1].record()
    torch.cuda.synchronize()
    return marks[0].elapsed_time(marks[count]), [marks[i].elapsed_time(marks[i + 1]) for i in range(count)]


def time_config(step, pool_len: int, warmup: int, min_steps: int = 200) -> dict:
    """Device time per step of one configuration: graphs of one step per pool buffer, at least
    `min_steps` steps and eight replays; median and 95th percentile over the replays."""
    import torch

    for i in range(max(warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    inner = pool_len if pool_len >= STEPS_PER_GRAPH else STEPS_PER_GRAPH * pool_len  # (whole passes over the pool)
    graph = capture(step, inner)
    replays = max(8, -(-min_steps // inner))
    graph.replay()
    total, each = timed_replays(lambda i: graph.replay(), replays)
    per_step = np.array(each) / inner
    return {"mean_ms": total / (replays * inner), "median_ms": float(np.median(per_step)),
            "p95_ms": float(np.percentile(per_step, 95)), "replays": replays, "steps_per_replay": inner}  # fmt: skip


def kernel_timeline(sampler, dw, replays: int = 7) -> dict:
    """Begin and end of each kernel of a step, in microseconds from the step's first begin: the
    kernels stamp the GPU's nanosecond timer (leat_sampler_time_kernels), here inside a replayed CUDA
    graph over up to 16 pool buffers, so the launches of a step overlap as they do when timed.
    Medians over the replays' last steps."""
    import torch

    sampler.time_kernels(True)
    for i in range(3):
        dw.step(sampler, i)
    torch.cuda.synchronize()
    graph = capture(lambda i: dw.step(sampler, i), min(len(dw.pool), 16))
    seen = []
    for _ in range(replays):
        graph.replay()
        seen.append(sampler.kernel_times())
    sampler.time_kernels(False)
    del graph
    names = [n for n in seen[-1] if all(n in s for s in seen[2:])]
    return {n: [round(float(np.median([s[n][j] for s in seen[2:]])) * 1e3, 2) for j in (0, 1)] for n in names}


def filter_microseconds(timeline: dict) -> float | None:
    span = timeline.get("filter_kernel")
    return None if span is None else max(span[1] - span[0], 1e-3)


def oracle_parity(w, ids, kept, cut, rows: int) -> dict:
    """The first `rows` rows of a result against the CPU oracle, by the parity rules of the tests:
    kept counts and cuts bit-exact, sampled ids identical unless the oracle marks the row as a
    nucleus-boundary tie (a float comparison within 1e-5 relative of flipping)."""
    from oracle import sampler_oracle as oracle

    sel = slice(0, rows)
    want = oracle.sample(w.logits[sel], w.options[sel], w.seed[sel], w.position[sel], history=w.history[sel],
                         penalties=w.penalties[sel], uniform_draws=w.uniform[sel], order="block", survivors=False)  # fmt: skip
    mismatch = fragile = 0
    for b in range(rows):
        same = ids[b] == want.ids[b, 0] and kept[b] == want.kept[b] and cut[b] == want.cut[b]
        if not same and want.margin[b] < 1e-5:
            fragile += 1
        elif not same:
            mismatch += 1
    return {"oracle_rows": rows, "oracle_mismatch": mismatch, "oracle_fragile": fragile}


def run_one(args) -> None:
    """One configuration, a few Python-launched steps: the command ncu captures are taken from."""
    import torch

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    kw = {"rows": args.rows} if args.rows and args.workload != 4 else {}
    w = workloads.CONFIGS[args.workload](**kw)
    sampler = Sampler(max(w.rows, 8), w.vocab, 256, device)
    dw = DeviceWorkload(w, device, min_pool_bytes=0, max_copies=1)
    step = (lambda i: sampler.argmax(dw.pool[0])) if args.op == "argmax" else (lambda i: dw.step(sampler, i))
    for i in range(args.warmup):
        step(i)
    total, _ = timed_replays(step, args.steps)
    print(json.dumps({"workload": WORKLOAD_NAMES[args.workload], "op": args.op, "rows": w.rows, "vocab": w.vocab,
                      "ms_per_step": total / args.steps,
                      "launch": dict(zip(("threads", "slices", "shared_bytes"),
                                         sampler.plan(w.rows, w.vocab, 0 if w.history is None else w.history.shape[1]))),
                      "kernels_per_step": sampler.last_launches}), flush=True)  # fmt: skip


def run_single(args) -> None:
    import torch

    from leat_b200 import sample as public_sample
    from leat_b200 import workloads
    from leat_b200.sampler import Sampler

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    peak, peak_kind = peak_hbm()
    sampler = Sampler(512, 262144, 256, device)

    # every configuration, device-timed under graph replay
    all_configs = {}
    headline = None
    for number, dtype in ((1, None), (2, None), (3, None), (4, None), (3, torch.bfloat16), (5, None)):
        w = workloads.CONFIGS[number]()
        dw = DeviceWorkload(w, device, dtype=dtype)
        timing = time_config(lambda i, dw=dw: dw.step(sampler, i), len(dw.pool), args.warmup)
        ms = timing["median_ms"]
        gbs = dw.logit_bytes / (ms * 1e-3) / 1e9
        launches_per_step = sampler.last_launches
        kernels = kernel_timeline(sampler, dw)
        filter_us = filter_microseconds(kernels)
        filter_gbs = None if filter_us is None else dw.logit_bytes / (filter_us * 1e-6) / 1e9
        all_configs[WORKLOAD_NAMES[number] + ("" if dtype is None else "_bf16_logits")] = {
            "rows": w.rows, "vocab": w.vocab, "us_per_step": round(ms * 1e3, 2), "p95_us": round(timing["p95_ms"] * 1e3, 2),
            "mean_us": round(timing["mean_ms"] * 1e3, 2), "replays": timing["replays"], "steps_per_replay": timing["steps_per_replay"],
            "rows_per_s": round(w.rows / (ms * 1e-3)), "launches_per_step": launches_per_step,
            "hbm_gbs": round(gbs, 1), "frac_of_measured": round(gbs / peak, 4), "frac_of_8tbs": round(gbs / NORTH_STAR_HBM_GBS, 4),
            "kernel_us": kernels,
            "filter_kernel_gbs": None if filter_gbs is None else round(filter_gbs, 1),
            "filter_kernel_frac_of_measured": None if filter_gbs is None else round(filter_gbs / peak, 4),
        }  # fmt: skip
        if dtype is None:
            # ops.argmax over the same logits (what leat's drafters run, leat/draft.py:166): one launch
            arg = time_config(lambda i, dw=dw: sampler.argmax(dw.pool[i % len(dw.pool)]), len(dw.pool), args.warmup)
            arg_gbs = dw.logit_bytes / (arg["median_ms"] * 1e-3) / 1e9
            all_configs[WORKLOAD_NAMES[number]]["argmax"] = {
                "us_per_call": round(arg["median_ms"] * 1e3, 2), "p95_us": round(arg["p95_ms"] * 1e3, 2),
                "hbm_gbs": round(arg_gbs, 1), "frac_of_measured": round(arg_gbs / peak, 4)}  # fmt: skip
        if number == HEADLINE:
            headline = (w, dw, kernels, launches_per_step)  # stays resident for the timed region below
        else:
            del dw
            torch.cuda.empty_cache()

    # the headline: exactly K steps of the largest configuration, one graph replay and one event each
    w, dw, kernels, launches_per_step = headline
    per_graph = steps_per_graph(args.steps)
    graph = capture(lambda i: dw.step(sampler, i), per_graph)
    single = capture(lambda i: dw.step(sampler, i), 1)
    for i in range(-(-args.warmup // per_graph)):
        graph.replay()
    with ClockSampler(device.index) as clocks:
        total, each = timed_replays(lambda i: graph.replay(), args.steps // per_graph)
        ms = total / args.steps
        each = [x / per_graph for x in each]
        keep_busy(lambda i: graph.replay(), ms * per_graph)
        single_total, _ = timed_replays(lambda i: single.replay(), args.steps)
        # end to end through the public call: host logits in pinned memory, copied in every step;
        # ids read back every step
        host_logits = torch.as_tensor(w.logits).pin_memory()
        host_ids = torch.empty((w.rows, 1), dtype=torch.int32).pin_memory()
        staging = torch.empty_like(dw.pool[0])

        def e2e_step(i):
            staging.copy_(host_logits, non_blocking=True)
            ids = public_sample(staging, dw.options, dw.seed, dw.position, history=dw.history,
                                penalties=dw.penalties, uniform=dw.uniform)  # fmt: skip
            host_ids.copy_(ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for i in range(3):
            e2e_step(i)
        e2e_total, _ = timed_replays(e2e_step, args.steps)
        ms_e2e = e2e_total / args.steps
    result = sampler.sample_full(dw.pool[0], dw.options, dw.seed, dw.position, history=dw.history, penalties=dw.penalties,
                                 uniform=dw.uniform, want_cut=True)  # fmt: skip
    torch.cuda.synchronize()
    parity = oracle_parity(w, result.ids.cpu().numpy().ravel(), result.kept.cpu().numpy(), result.cut.cpu().numpy(),
                           CPU_SAMPLE_ROWS)  # fmt: skip
    parity.update({"rows": w.rows, "mismatch": parity["oracle_mismatch"], "fragile": parity["oracle_fragile"],
                   "status_word": int(result.status.item())})  # fmt: skip
    value = w.rows / (ms * 1e-3)
    achieved = w.logit_bytes / (ms * 1e-3) / 1e9  # the whole call: every launch of a step
    filter_us = filter_microseconds(kernels)
    filter_gbs = w.logit_bytes / (filter_us * 1e-6) / 1e9
    threads = os.cpu_count() or 1
    cpu_value, cpu_sample = cpu_rows_per_second(workloads.CONFIGS[HEADLINE](rows=CPU_SAMPLE_ROWS), "U", seconds=12.0, threads=threads)
    line = {
        "metric": "sampler rows/s", "value": value, "unit": "rows/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "median_ms": float(np.median(each)), "p95_ms": float(np.percentile(each, 95)),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(1, w.vocab),
        "steps_per_graph": per_graph, "ms_per_step_one_step_per_graph": single_total / args.steps,
        "notes": {"l2": dw.l2_note,
                  "timing": "CUDA events on the launching stream: one before the K steps, one after each replay of a CUDA graph "
                            f"holding {per_graph} consecutive leat_sample calls (a decode graph holds the model's kernels around "
                            "the sampler's; the graph's own launch is the engine's cost); ms_per_step = region / K, median and "
                            "p95 over the replays, per step"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE * w.logit_bytes, "peak_kind": peak_kind,
                     "kernel": "the whole call: filter_kernel, finish_list_kernel, sample_kernel",
                     "algorithmic_bytes_per_launch": w.logit_bytes, "launch_us": ms * 1e3,
                     "frac_of_8tbs": achieved / NORTH_STAR_HBM_GBS,
                     "filter_kernel": {"achieved": filter_gbs, "frac": filter_gbs / peak, "launch_us": filter_us,
                                       "note": "the kernel that moves the bytes: its last block's end minus its first block's "
                                               "begin on the GPU's timer, inside a replayed graph (it works the rows' floors out too)"},
                     "kernel_us": kernels,
                     "kernel_us_note": "begin and end of each kernel of a step from the step's first begin; the launches overlap "
                                       "(each is a programmatic dependent of the one before)"},
        "cpu_baseline": {"value": cpu_value, "unit": "rows/s", "cores": threads, "kind": "port", "sample": cpu_sample},
        "e2e": {"value": w.rows / (ms_e2e * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": w.logit_bytes,
                "d2h_bytes_per_step": w.rows * 4},
        "parity": parity, "gpu_launches": launches_per_step * args.steps, "clocks": clocks.summary(), "all_configs": all_configs,
        "us_per_step_b1": all_configs[WORKLOAD_NAMES[1]]["us_per_step"],
    }  # fmt: skip
    print(json.dumps(line), flush=True)
    if parity["mismatch"]:
        sys.exit(3)


def run_sharded(args) -> None:
    import torch
    import torch.distributed as dist

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler
    from leat_b200.sharded import ShardedSampler

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    peak, peak_kind = peak_hbm()
    w = workloads.CONFIGS[HEADLINE]()
    sharded = ShardedSampler(w.rows, w.vocab, k_max=64, cap=128, device=device)
    start, stop = sharded.start, sharded.stop
    t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
    slice_bytes = (stop - start) * w.rows * 4
    copies = 1 if slice_bytes > L2_BYTES else min(32, -(-2 * L2_BYTES // slice_bytes))
    base = torch.as_tensor(np.ascontiguousarray(w.logits[:, start:stop])).to(device)
    pool = [base] + [base.clone() for _ in range(copies - 1)]
    options, penalties, history, uniform, position = t(w.options), t(w.penalties), t(w.history), t(w.uniform), t(w.position)
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    out = torch.empty((w.rows, 1), dtype=torch.int32, device=device)

    def step(i):
        return sharded.sample(pool[i % len(pool)], options, seed, position, history=history, penalties=penalties,
                              uniform=uniform, out=out)  # fmt: skip

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    per_graph = steps_per_graph(args.steps)
    replay, how = sharded.replayable(pool, options, seed, position, history, penalties, uniform, out, per_graph)
    for i in range(3):
        replay(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        total, each = timed_replays(replay, args.steps // per_graph)
        each = [x / per_graph for x in each]
        stats = torch.tensor([total / args.steps, float(np.median(each)), float(np.percentile(each, 95))], device=device)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        ms, median_ms, p95_ms = (float(x) for x in stats.tolist())
        keep_busy(replay, ms * per_graph)
    dist.barrier()
    torch.cuda.synchronize()
    replayed_ids = out.clone()  # what the last of the replayed steps left (checked below)
    # end to end: this rank's slice comes from pinned host memory every step, the ids go back
    host_slice = torch.as_tensor(np.ascontiguousarray(w.logits[:, start:stop])).pin_memory()
    host_ids = torch.empty((w.rows, 1), dtype=torch.int32).pin_memory()

    def e2e_step(i):
        pool[0].copy_(host_slice, non_blocking=True)
        result = sharded.sample(pool[0], options, seed, position, history=history, penalties=penalties, uniform=uniform, out=out)
        host_ids.copy_(result.ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    dist.barrier()
    torch.cuda.synchronize()
    e2e_total, _ = timed_replays(e2e_step, args.steps)
    ms_e2e = torch.tensor([e2e_total / args.steps], device=device)
    dist.all_reduce(ms_e2e, op=dist.ReduceOp.MAX)
    ms_e2e = float(ms_e2e.item())

    # parity, outside the timed regions: one more step on every rank (it holds the exchange); every
    # rank's ids must be the same; rank 0 compares them with the one-GPU sampler on the whole logits
    # (all rows: ids, survivor counts, cuts) and with the CPU oracle on the first rows
    result = sharded.sample(pool[0], options, seed, position, history=history, penalties=penalties, uniform=uniform)
    torch.cuda.synchronize()
    everyone = [torch.empty_like(result.ids) for _ in range(world)]
    dist.all_gather(everyone, result.ids.contiguous())
    # (every step had the same inputs: the last replayed step must have given the same ids)
    stale = (replayed_ids != result.ids).sum().to(torch.int64)
    dist.all_reduce(stale)
    parity = None
    if rank == 0:
        ids = result.ids.cpu().numpy().ravel()
        kept, cut = result.kept.cpu().numpy(), result.cut.cpu().numpy()
        differing_ranks = sum(int(not torch.equal(everyone[0], other)) for other in everyone[1:])
        single = Sampler(w.rows, w.vocab, 64, device)
        one = single.sample_full(torch.as_tensor(w.logits).to(device), options, seed, position, history=history,
                                 penalties=penalties, uniform=uniform, want_cut=True)  # fmt: skip
        torch.cuda.synchronize()
        vs_one = int(np.count_nonzero((ids != one.ids.cpu().numpy().ravel()) | (kept != one.kept.cpu().numpy())
                                      | (cut != one.cut.cpu().numpy())))  # fmt: skip
        parity = oracle_parity(w, ids, kept, cut, CPU_SAMPLE_ROWS)
        parity.update({"rows": w.rows, "ranks_differing": differing_ranks, "rows_differing_from_one_gpu": vs_one,
                       "ids_differing_after_replays": int(stale.item()),
                       "mismatch": parity["oracle_mismatch"] + vs_one + differing_ranks + int(stale.item()),
                       "fragile": parity["oracle_fragile"],
                       "status_word": int(result.status.item())})  # fmt: skip
        del single, one
        achieved = w.logit_bytes / world / (ms * 1e-3) / 1e9  # per GPU: each reads its slice once
        line = {
            "metric": "sampler rows/s", "value": w.rows / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "median_ms": median_ms, "p95_ms": p95_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": headline_config(world, w.vocab), "steps_per_graph": per_graph,
            "notes": {"l2": f"logits pool of {len(pool)} buffers per rank cycled, larger than L2" if len(pool) > 1
                      else "each rank's slice is larger than L2",
                      "exchange": sharded.exchange_note,
                      "timing": "CUDA events on the launching stream: one before the K steps, one after each; " + how +
                                "; every figure is the max over ranks"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind,
                         "kernel": "the whole step per GPU (floor, filter, candidates, exchange, finish) over its vocabulary slice",
                         "algorithmic_bytes_per_launch": w.logit_bytes // world, "launch_us": ms * 1e3},
            "e2e": {"value": w.rows / (ms_e2e * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": int(host_slice.numel() * 4) * world,
                    "d2h_bytes_per_step": w.rows * 4 * world},
            "parity": parity, "gpu_launches": sharded.launches_per_step * args.steps, "clocks": clocks.summary(),
        }  # fmt: skip
        print(json.dumps(line), flush=True)
    bad = torch.tensor([int(bool(parity and parity["mismatch"]))], device=device)
    dist.broadcast(bad, 0)
    del replay
    torch.cuda.synchronize()
    dist.barrier()
    sharded.close()
    dist.destroy_process_group()
    if int(bad.item()):
        sys.exit(3)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", type=int, default=0, choices=[0, 1, 2, 3, 4, 5],
                        help="profiling aid: time only this configuration, launched from Python, and print a short line")
    parser.add_argument("--rows", type=int, default=0, help="with --workload: fewer rows than the configuration has")
    parser.add_argument("--op", default="sample", choices=["sample", "argmax"],
                        help="with --workload: the sampler's step (default) or ops.argmax over the same logits")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)
    if args.workload:
        run_one(args)
    elif args.impl == "reference":
        run_reference(args)
    elif int(os.environ.get("WORLD_SIZE", 1)) > 1:
        run_sharded(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
